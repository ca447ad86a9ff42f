"""Comparison helpers with the reference's tolerance metric (triton_kernels/testing.py:18-88)."""
import torch


def assert_equal(ref, tri):
    if isinstance(ref, torch.Tensor):
        assert torch.all(ref == tri)
    else:
        assert ref == tri


def assert_close(ref, tri, maxtol=None, rmstol=None, description="--", verbose=True):
    """Both tensors are normalised by max|ref|; the element error is |ref - tri| / max(rms(ref), |ref|);
    its maximum must stay below `maxtol` (default 2e-2) and its RMS below `rmstol` (default 4e-3)."""
    if tri.dtype.itemsize == 1:
        ref_as_type = ref.to(tri.dtype)
        if ref.dtype == tri.dtype:
            assert torch.all(ref_as_type == tri)
            return
        ref = ref_as_type
    if ref.numel() == 0:
        return
    maxtol = 2e-2 if maxtol is None else maxtol
    rmstol = 4e-3 if rmstol is None else rmstol
    ref = ref.to(torch.float32).detach()
    tri = tri.to(torch.float32).detach()
    assert ref.shape == tri.shape, f"Tensors must have same size {ref.shape=} {tri.shape=}"
    inf_ref, inf_tri = torch.isinf(ref), torch.isinf(tri)
    assert torch.equal(inf_ref, inf_tri), "Tensor must have same infinite elements"
    refn = torch.where(inf_ref, 0, ref)
    trin = torch.where(inf_tri, 0, tri)
    eps = 1.0e-30
    mult = 1.0 / (torch.max(torch.abs(refn)) + eps)
    refn, trin = refn * mult, trin * mult
    ref_rms = torch.sqrt(torch.square(refn).mean()) + eps
    rel_err = torch.abs(refn - trin) / torch.maximum(ref_rms, torch.abs(refn))
    max_err = torch.max(rel_err).item()
    rms_err = torch.sqrt(torch.square(rel_err).mean()).item()
    if verbose:
        print(f"{description} maximum relative error = {max_err} (threshold = {maxtol})")
        print(f"{description} RMS relative error = {rms_err} (threshold = {rmstol})")
    assert max_err <= maxtol
    assert rms_err <= rmstol


def make_synthetic_layer(n_expts, d_model, d_ff, device, seed=0, keep_canonical=False, chunk=8, block_scaled=False,
                         layouts=True):
    """Random-init MoE expert weights of a gpt-oss-shaped layer: bf16 N(0, 0.02) quantised to MXFP4 along K,
    bias bf16 N(0, 0.01).  Experts are generated and quantised `chunk` at a time to bound peak memory.
    `block_scaled` adds a second copy in the layouts of the block-scaled kernel (used for steps with few rows per
    expert).  `layouts=False` skips every re-layout and returns the canonical tensors only (a checker that wants the
    very weights another process generated from the same seed)."""
    from .moe import MoeLayerWeights
    from .numerics_details.mxfp import downcast_to_mxfp
    from .tensor import FP4, convert_layout, wrap_torch_tensor
    from .tensor_details.layout import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout,
                                        make_default_matmul_mxfp4_w_layout, make_default_matmul_mxfp4_w_scale_layout)
    g = torch.Generator(device=device).manual_seed(seed)

    def quant(K, N):
        qs, ss = [], []
        for e0 in range(0, n_expts, chunk):
            n = min(chunk, n_expts - e0)
            w = (torch.randn(n, K, N, device=device, generator=g) * 0.02).bfloat16()
            q, s = downcast_to_mxfp(w, torch.uint8, axis=1)
            qs.append(q)
            ss.append(s)
        q = torch.cat([t.transpose(1, 2) for t in qs]).transpose(1, 2)          # keeps K contiguous
        s = torch.cat([t.transpose(1, 2) for t in ss]).transpose(1, 2)
        tq = ts = bq = bs = None
        if layouts:
            tq = convert_layout(wrap_torch_tensor(q, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=-2))
            ts = convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=-2))
        if block_scaled and layouts:
            bq = convert_layout(wrap_torch_tensor(q, dtype=FP4), B200BlockScaledValueLayout())
            bs = convert_layout(wrap_torch_tensor(s), B200BlockScaledScaleLayout())
        keep = keep_canonical or not layouts
        return tq, ts, (q if keep else None), (s if keep else None), bq, bs

    w1, s1, q1, c1, bq1, bs1 = quant(d_model, 2 * d_ff)
    w2, s2, q2, c2, bq2, bs2 = quant(d_ff, d_model)
    b1 = (torch.randn(n_expts, 2 * d_ff, device=device, generator=g) * 0.01).bfloat16()
    b2 = (torch.randn(n_expts, d_model, device=device, generator=g) * 0.01).bfloat16()
    return MoeLayerWeights(w1, s1, b1, w2, s2, b2, w1_q=q1, w1_s=c1, w2_q=q2, w2_s=c2,
                           w1_bs=bq1, w1_bs_scale=bs1, w2_bs=bq2, w2_bs_scale=bs2)
