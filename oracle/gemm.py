"""CPU oracle for the ragged grouped GEMM, SwiGLU, the top-k combine and the whole MoE layer
(TEST INFRASTRUCTURE ONLY).

Follows, in the reference's ``triton_kernels`` package: ``matmul.py:772-817``
(``apply_precision``: MXFP4 weights are dequantised to bf16 first), ``matmul.py:840-931``
(``matmul_torch``), ``swiglu.py:89-100`` (``swiglu_torch``), ``reduce.py:1181-1214``
(``reduce_torch``) and the layer composition of ``tests/test_distributed.py:203-220`` /
``bench/bench_mlp.py:60-96``.
"""
import torch

from .mxfp import upcast_from_mxfp_oracle
from .routing import topk_oracle, bitmatrix_metadata_oracle


def dequant_weight_oracle(w_q: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """[E, K/2, N] packed e2m1 + [E, K/32, N] e8m0 -> [E, K, N] bf16 (matmul.py:795-808, mx axis = -2)."""
    return upcast_from_mxfp_oracle(w_q, w_scale, torch.bfloat16, axis=-2)


def matmul_oracle(x, w, bias=None, slice_sizes=None, gather_indx=None, scatter_indx=None,
                  betas=None, gammas=None, out_dtype=None):
    """Ragged grouped GEMM: rows ``[off_e, off_e + size_e)`` of the (gathered) activations are multiplied
    by ``w[e]``; fp32 accumulation; ``(acc + bias[e] * betas) * gammas``; rows are rounded to the
    activation dtype and optionally scattered (matmul.py:891-927).

    x [M, K] float; w [E, K, N] float (already dequantised); bias [E, N] or None;
    slice_sizes [E] int or None (then E must be 1 and all rows belong to slice 0).
    Rows beyond ``sum(slice_sizes)`` stay zero, as in the reference's oracle.
    """
    out_dtype = out_dtype or x.dtype
    E, K, N = w.shape
    n_rows = x.shape[0] if gather_indx is None else gather_indx.shape[0]
    if slice_sizes is None:
        assert E == 1
        bounds = [(0, n_rows)]
    else:
        offs = [0]
        for s in slice_sizes.tolist():
            offs.append(offs[-1] + int(s))
        bounds = list(zip(offs[:-1], offs[1:]))
    y = torch.zeros((n_rows, N), dtype=out_dtype)
    xf = x.float()
    for e, (lo, hi) in enumerate(bounds):
        if hi <= lo:
            continue
        rows = torch.arange(lo, hi) if gather_indx is None else gather_indx[lo:hi].long()
        acc = xf[rows] @ w[e].float()
        if bias is not None:
            b = bias[e].float()
            acc = acc + (b if betas is None else b * betas[lo:hi, None].float())
        if gammas is not None:
            acc = acc * gammas[lo:hi, None].float()
        y[lo:hi] = acc.to(out_dtype)
    if scatter_indx is None:
        return y
    out = torch.zeros((scatter_indx.shape[0], N), dtype=out_dtype)
    m = scatter_indx != -1
    out[scatter_indx[m].long()] = y[m]
    return out


def swiglu_oracle(a: torch.Tensor, alpha: float, limit=None) -> torch.Tensor:
    """Interleaved SwiGLU: even columns are the gate, odd columns the linear branch (swiglu.py:89-100)."""
    g = a[..., 0::2]
    l = a[..., 1::2]
    if limit is not None:
        g = g.clamp(max=limit)
        l = l.clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g)) * (l + 1)


def reduce_oracle(x: torch.Tensor, dim: int, mask=None, scale=None) -> torch.Tensor:
    """``sum over dim of where(mask, x * scale, 0)`` in fp32, cast back to x.dtype (reduce.py:1181-1214)."""
    xf = x.float()
    if scale is not None:
        xf = xf * scale.float()
    if mask is not None:
        xf = torch.where(mask.bool(), xf, torch.zeros((), dtype=torch.float32))
    return xf.sum(dim=dim).to(x.dtype)


def moe_layer_oracle(x, logits, w1, b1, w2, b2, k, alpha, limit, fuse_activation_fp32=False):
    """One MoE layer: routing -> fc1 (+bias) -> SwiGLU -> fc2 (+bias, * routing weight) -> combine.

    w1 [E, K, 2F], w2 [E, F, K] are dequantised float weights.  fc2's epilogue multiplies
    ``acc + bias`` by the routing weight of the row (``gammas`` in expert-sorted order); the combine
    sums the k expert outputs of each token (test_distributed.py:213-220 with ``gammas``).
    With ``fuse_activation_fp32`` the SwiGLU sees the fp32 accumulator instead of the bf16-rounded
    fc1 output (what a fused epilogue does); both are inside the GEMM tolerance.
    """
    T, E = logits.shape
    vals, indx, _ = topk_oracle(logits, k, apply_softmax=True)
    col_sum, col_sorted, row_sorted = bitmatrix_metadata_oracle(indx, E)
    gather = torch.div(col_sorted, k, rounding_mode="trunc")
    gam = vals.reshape(-1)[col_sorted.long()].float()
    h = matmul_oracle(x, w1, b1, col_sum, gather_indx=gather,
                      out_dtype=torch.float32 if fuse_activation_fp32 else x.dtype)
    h = swiglu_oracle(h.float(), alpha, limit).to(x.dtype)
    y = matmul_oracle(h, w2, b2, col_sum, scatter_indx=col_sorted, gammas=gam)
    return reduce_oracle(y.view(T, k, -1), dim=1)


def moe_layer_tokens_oracle(x_rows, logits_rows, expert_weights, k, alpha, limit, h_dtype=None, out_dtype=None):
    """The layer of ``moe_layer_oracle`` for a few token rows of a large problem, without materialising every
    expert: ``expert_weights(e) -> (w1 [K, 2F], b1 [2F], w2 [F, K], b2 [K])`` returns the dequantised weights of
    expert ``e`` (float tensors) and is called once per expert the rows are routed to.

    Same steps and roundings as ``moe_layer_oracle``: top-k + softmax over the selected logits (topk.py:144-185),
    fc1 + bias in fp32 rounded to the activation dtype, SwiGLU (swiglu.py:89-100) rounded to the activation
    dtype, fc2 + bias times the routing weight rounded to the activation dtype (matmul.py:891-927), then the
    k-way sum in fp32 rounded once (reduce.py:1181-1214).

    With ``h_dtype`` (e.g. ``torch.float8_e4m3fn``: e4m3 activations between the two GEMMs, the reference's fp8 mode) the
    SwiGLU sees the fp32 accumulator and its result is rounded to ``h_dtype``; ``x_rows`` may then be any float dtype
    holding the (already quantised) inputs and ``out_dtype`` names the dtype of fc2's rows."""
    T = x_rows.shape[0]
    vals, indx, _ = topk_oracle(logits_rows, k, apply_softmax=True)
    dt = out_dtype or x_rows.dtype
    y = torch.zeros((T, k, x_rows.shape[1]), dtype=dt)
    cache = {}
    for t in range(T):
        for j in range(k):
            e = int(indx[t, j])
            if e not in cache:
                cache[e] = [w.float() for w in expert_weights(e)]
            w1, b1, w2, b2 = cache[e]
            if h_dtype is None:
                h = (x_rows[t].float() @ w1 + b1).to(dt)
                h = swiglu_oracle(h.float(), alpha, limit).to(dt)
            else:
                h = swiglu_oracle(x_rows[t].float() @ w1 + b1, alpha, limit).to(h_dtype)
            y[t, j] = ((h.float() @ w2 + b2) * vals[t, j].float()).to(dt)
    return reduce_oracle(y, dim=1)
