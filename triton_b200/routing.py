"""`routing()`: the composition the reference's earlier API exposed under this name, written out in
its tests today (python/triton_kernels/tests/test_distributed.py:203-210)."""
import torch

from . import _lib
from .tensor import BIT, BitmatrixMetadata, RaggedTensorMetadata, SparseMatrix, make_ragged_tensor_metadata, wrap_torch_tensor
from .tensor_details.ragged_tensor import _empty_aligned
from .topk import topk


FUSED_MAX_TOKENS = 1 << 22


def route(logits, n_expts_act, apply_softmax=True):
    """Top-k, expert histogram, expert-major sort and ragged metadata of one batch of logits in three launches
    (`moe_route`): -> (ragged_metadata, sparse_logits), the same objects `topk` + `make_ragged_tensor_metadata` return.
    More than 256 experts, more than FUSED_MAX_TOKENS tokens, or logits that are not a plain 2-D tensor take the
    five-launch composition of the separate entry points."""
    if not (isinstance(logits, torch.Tensor) and logits.ndim == 2 and logits.shape[1] <= 256
            and 0 < logits.shape[0] <= FUSED_MAX_TOKENS and logits.stride(1) == 1):
        sparse = topk(logits, n_expts_act, apply_softmax=apply_softmax)
        md = sparse.mask_metadata
        return make_ragged_tensor_metadata(md.col_sum, md.row_sorted_indx.shape[0]), sparse
    lib = _lib.load()
    T, E = logits.shape
    k = n_expts_act
    dev = logits.device
    vals = torch.empty((T, k), dtype=logits.dtype, device=dev)
    indx = torch.empty((T, k), dtype=torch.int16, device=dev)
    words, t_pad = (E + 31) // 32, (T + 31) // 32 * 32
    bm_store = torch.empty((words, t_pad), dtype=torch.int32, device=dev)
    bm = bm_store.transpose(0, 1)[:T]
    col_sum = torch.empty(E, dtype=torch.int32, device=dev)
    combined = torch.empty(2 * T * k, dtype=torch.int32, device=dev)
    col_sorted, row_sorted = combined[: T * k], combined[T * k:]
    mnb = RaggedTensorMetadata.max_n_blocks(E, T * k)
    offs = _empty_aligned((5, E + 1), dev)
    sched = _empty_aligned((4, mnb), dev)
    slice_offs, block_offs = offs[0], offs[1:]
    ws_bytes = lib.moe_route_workspace(T, E, k)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    _lib.check(lib.moe_route(_lib.ptr(logits), _lib.dtype_code(logits.dtype), T, E, k, int(bool(apply_softmax)), logits.stride(0),
                             _lib.ptr(vals), vals.stride(0), _lib.ptr(indx), indx.stride(0), _lib.ptr(bm), bm.stride(0),
                             bm.stride(1), _lib.ptr(col_sum), _lib.ptr(col_sorted), _lib.ptr(row_sorted), _lib.ptr(slice_offs),
                             _lib.ptr(block_offs), block_offs.stride(0), _lib.ptr(sched), sched.stride(0), mnb, _lib.ptr(ws),
                             ws_bytes, _lib.stream()), "moe_route")
    bitmatrix = wrap_torch_tensor(bm, dtype=BIT, shape=[T, E], shape_max=[T, None])
    sparse = SparseMatrix(indx=indx, vals=vals, mask=bitmatrix,
                          mask_metadata=BitmatrixMetadata(col_sum=col_sum, col_sorted_indx=col_sorted, row_sorted_indx=row_sorted))
    return RaggedTensorMetadata(col_sum, slice_offs, block_offs, sched), sparse


def routing(logits, n_expts_act, all_gather=False, y_indx=None, symm_mem_pool=None, apply_softmax=True):
    """-> (ragged_metadata, gather_idx, scatter_idx, sparse_logits).

    gather_idx[p] is the token whose activations feed expert-sorted row p, scatter_idx[p] the flat
    (token * k + slot) row its output goes to; sparse_logits.vals holds the routing weights."""
    if not all_gather and y_indx is None:
        ragged, sparse = route(logits, n_expts_act, apply_softmax)
        combine_indx = sparse.mask_metadata.col_sorted_indx
    else:
        sparse = topk(logits, n_expts_act, apply_softmax=apply_softmax, all_gather=all_gather, y_indx=y_indx,
                      symm_mem_pool=symm_mem_pool)
        dispatch_indx = sparse.mask_metadata.row_sorted_indx
        combine_indx = sparse.mask_metadata.col_sorted_indx
        ragged = make_ragged_tensor_metadata(sparse.mask_metadata.col_sum, dispatch_indx.shape[0])
    gather_idx = torch.div(combine_indx, n_expts_act, rounding_mode="trunc")
    scatter_idx = combine_indx
    return ragged, gather_idx, scatter_idx, sparse
