"""CPU oracle for routing: top-k, expert bitmatrix, histogram, stable expert sort and
ragged-segment metadata (TEST INFRASTRUCTURE ONLY).

Follows, in the reference's ``triton_kernels`` package:
``topk.py:144-185`` (``topk_torch``) with the tie-break of
``topk_details/_topk_forward.py:27-35`` (equal values -> smaller expert index);
``tensor_details/bitmatrix.py:157-168`` (``make_bitmatrix_metadata_torch``) with the
flat-index semantics of the kernel at ``bitmatrix.py:43-73``;
``tensor_details/ragged_tensor.py:217-253`` and ``:388-433``.
"""
import numpy as np
import torch

BLOCK_SIZES = (16, 32, 64, 128)            # ragged_tensor.py:83-89 (NVIDIA)


def n_blocks(n_slices: int, n_total_rows: int, block_size: int) -> int:
    """Upper bound on the number of row blocks (ragged_tensor.py:73-77)."""
    if n_total_rows <= n_slices:
        return n_total_rows
    return n_slices - 1 - ((n_slices - n_total_rows - 1) // block_size)


def max_n_blocks(n_slices: int, n_total_rows: int) -> int:
    return n_blocks(n_slices, n_total_rows, min(BLOCK_SIZES))


def topk_oracle(logits: torch.Tensor, k: int, apply_softmax: bool = True, y_indx=None, n_rows=None):
    """-> (vals [T,k] logits.dtype, indx [T,k] int32 (-1 for rows >= n_rows), bitmatrix int32 [T, ceil(E/32)]).

    Selection is by (value descending, index ascending); the selected k are output
    in that order; softmax runs in fp32 over the selected k and is cast back
    (topk.py:153-172).  When `y_indx` is given, selection is skipped and values are
    gathered at those indices, keeping their order (topk.py:162-171).
    """
    T, E = logits.shape
    n_rows = T if n_rows is None else int(n_rows)
    x = logits
    if y_indx is None:
        order = torch.argsort(-x.float(), dim=1, stable=True)[:, :k]
    else:
        order = y_indx.long()
    vals = torch.take_along_dim(x[:n_rows], order[:n_rows], dim=1)
    if apply_softmax:
        vals = torch.softmax(vals.float(), dim=-1).to(x.dtype)
    vals = torch.cat([vals, x[n_rows:, :k]], dim=0)
    indx = order.to(torch.int32).clone()
    indx[n_rows:] = -1
    words = (E + 31) // 32
    bm = np.zeros((T, words), np.uint32)
    ii = indx.numpy()
    for s in range(k):
        col = ii[:n_rows, s].astype(np.int64)
        np.bitwise_or.at(bm, (np.arange(n_rows), col // 32), (np.uint32(1) << (col % 32).astype(np.uint32)))
    return vals, indx, torch.from_numpy(bm.view(np.int32))


def router_topk_oracle(x: torch.Tensor, wg: torch.Tensor, bg, k: int, apply_softmax: bool = True, logits_dtype=None):
    """The router of the reference's MoE layer: `logits = matmul(x, wg, bg)` (bench/bench_mlp.py:70; fp32 accumulation,
    bias added in fp32, result cast to the activation dtype: matmul.py:772-931) followed by `topk` (topk.py:144-185).
    -> (logits in `logits_dtype` (default x.dtype), vals, indx, bitmatrix) with the last three as `topk_oracle` gives them."""
    logits_dtype = x.dtype if logits_dtype is None else logits_dtype
    logits = x.float() @ wg.float()
    if bg is not None:
        logits = logits + bg.float()
    logits = logits.to(logits_dtype)
    vals, indx, bm = topk_oracle(logits, k, apply_softmax)
    return logits, vals, indx, bm


def bitmatrix_metadata_oracle(indx: torch.Tensor, n_expts: int):
    """indx [T,k] (int, -1 = dropped) -> (col_sum [E], col_sorted_indx [T*k], row_sorted_indx [T*k]), int32.

    Stable counting sort of the flat entries ``i = token*k + slot`` by expert:
    ``row_sorted_indx[i]`` = position of entry i in expert-major order,
    ``col_sorted_indx`` = its inverse; dropped entries are skipped and both arrays
    are padded with -1 (bitmatrix.py:43-73, 157-168).
    """
    flat = indx.reshape(-1).to(torch.int64).numpy()
    n = flat.shape[0]
    keep = np.nonzero(flat >= 0)[0]
    order = keep[np.argsort(flat[keep], kind="stable")]
    col_sorted = np.full(n, -1, np.int32)
    row_sorted = np.full(n, -1, np.int32)
    col_sorted[: order.shape[0]] = order
    row_sorted[order] = np.arange(order.shape[0], dtype=np.int32)
    col_sum = np.bincount(flat[keep], minlength=n_expts).astype(np.int32)[:n_expts]
    return torch.from_numpy(col_sum), torch.from_numpy(col_sorted), torch.from_numpy(row_sorted)


def ragged_metadata_oracle(slice_sizes: torch.Tensor, n_total_rows: int):
    """-> (slice_offs [E+1], block_offs [4,E+1], block_schedule [4,max_n_blocks]) int32 (ragged_tensor.py:217-253).

    ``block_schedule[b][block_offs[b][e] + j] = (j << 16) | e``, padded with -1.
    """
    sizes = slice_sizes.to(torch.int64).numpy()
    E = sizes.shape[0]
    mnb = max_n_blocks(E, n_total_rows)
    slice_offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    block_offs = np.zeros((len(BLOCK_SIZES), E + 1), np.int32)
    sched = np.full((len(BLOCK_SIZES), mnb), -1, np.int32)
    for b, bs in enumerate(BLOCK_SIZES):
        nb = (sizes + bs - 1) // bs
        block_offs[b] = np.concatenate([[0], np.cumsum(nb)])
        ent = [np.int64(j << 16) | e for e in range(E) for j in range(int(nb[e]))]
        ent = np.array(ent[:mnb], np.int64).astype(np.int32)
        sched[b, : ent.shape[0]] = ent
    return torch.from_numpy(slice_offs), torch.from_numpy(block_offs), torch.from_numpy(sched)


def remap_ragged_metadata_oracle(slice_sizes, slice_offs, block_offs, block_schedule, slice_map):
    """Restrict ragged metadata to the slices with ``slice_map[e] != -1`` (ragged_tensor.py:388-433).

    Surviving entries keep their order and their *global* offsets; slice ids in the
    schedule are rewritten through `slice_map`; tails are padded with -1 and the
    number of surviving blocks is stored at ``block_offs[b][n_surviving]``.
    """
    smap = slice_map.to(torch.int64).numpy()
    keep = smap != -1
    E = keep.shape[0]

    def compact(v, m):
        v = np.asarray(v)
        return np.concatenate([v[m], np.full(int((~m).sum()), -1, v.dtype)])

    keep1 = np.concatenate([keep, [False]])
    out_sizes = compact(slice_sizes.numpy(), keep)
    out_offs = compact(slice_offs.numpy(), keep1)
    bo, bs = [], []
    for b in range(block_offs.shape[0]):
        o = compact(block_offs[b].numpy(), keep1)
        s = block_schedule[b].numpy().view(np.uint32).astype(np.int64)     # 0 .. 2^32-1, padding = 0xFFFFFFFF
        sid = s & 0xFFFF
        valid = sid != 0xFFFF
        m = np.zeros(s.shape, bool)
        m[valid] = smap[sid[valid]] != -1
        kept = s[m]
        out = np.full(s.shape, 0xFFFFFFFF, np.int64)
        out[: kept.shape[0]] = (kept & 0xFFFF0000) | smap[kept & 0xFFFF]
        o[int(keep.sum())] = kept.shape[0]
        bo.append(o)
        bs.append(out.astype(np.uint32).view(np.int32))
    assert E + 1 == out_offs.shape[0]
    return (torch.from_numpy(out_sizes.astype(np.int32)), torch.from_numpy(out_offs.astype(np.int32)),
            torch.from_numpy(np.stack(bo).astype(np.int32)), torch.from_numpy(np.stack(bs).astype(np.int32)))
