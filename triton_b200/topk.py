"""Top-k expert selection (+ softmax over the selected logits) and the expert bitmatrix
(triton_kernels/topk.py:25-141).  Forward only."""
from typing import Optional, Union

import torch

from . import _lib
from .tensor import BIT, SparseMatrix, Tensor, wrap_torch_tensor


def topk_forward(x, k, apply_softmax=True, dim=1, y_indx=None, n_rows=None, all_gather=False, symm_mem_pool=None):
    """-> (y_vals [T,k] x.dtype, y_indx [T,k] int16, bitmatrix BIT Tensor [T, E]).

    The bitmatrix is stored transposed, uint32 [ceil(E/32), ceil32(T)], and viewed as [T, words] with
    strides (1, ceil32(T)) exactly as topk.py:52-57 lays it out.  With `all_gather` every rank's rows
    are gathered (rank-major) through the pool's process group after the local kernel.
    """
    lib = _lib.load()
    if isinstance(x, Tensor):
        n_rows_arg, x_t = x.shape[0], x.storage.data
        n_rows = n_rows_arg if n_rows is None else n_rows
        x = x_t
    assert x.ndim == 2 and dim == 1
    assert x.shape[-1] < 32768
    assert symm_mem_pool is not None or not all_gather
    T, E = x.shape
    dev = x.device
    if x.stride(1) != 1:
        x = x.contiguous()
    use_provided = y_indx is not None
    world = symm_mem_pool.mesh.world_size if all_gather else 1
    rank = symm_mem_pool.mesh.local_rank if all_gather else 0
    T_out = T * world
    y_vals = torch.empty((T_out, k), dtype=x.dtype, device=dev)
    if y_indx is None:
        y_indx_full = torch.empty((T_out, k), dtype=torch.int16, device=dev)
    else:
        y_indx_full = y_indx if y_indx.dtype == torch.int16 else y_indx.to(torch.int16)
        assert y_indx_full.shape[0] >= T_out and y_indx_full.stride(1) == 1
    words = (E + 31) // 32
    t_pad = (T_out + 31) // 32 * 32
    bm_store = torch.empty((words, t_pad), dtype=torch.int32, device=dev)
    bm = bm_store.transpose(0, 1)[:T_out]
    n_rows_dev = None
    if n_rows is not None:
        if isinstance(n_rows, torch.Tensor):
            n_rows_dev = n_rows.to(torch.int32)
        elif int(n_rows) < T:
            n_rows_dev = torch.tensor([int(n_rows)], dtype=torch.int32, device=dev)
    r0 = rank * T
    vals_loc, indx_loc, bm_loc = y_vals[r0:r0 + T], y_indx_full[r0:r0 + T], bm[r0:r0 + T]
    # with peer-mapped routing buffers the kernel writes this rank's rows straight into them: the all-gather then reads
    # every rank's rows (this one's included) from there and no copy runs in between
    direct = (all_gather and world > 1 and not use_provided and getattr(symm_mem_pool, "peer_ok", False)
              and x.dtype == torch.float32 and symm_mem_pool.peer_shape[0] == T and symm_mem_pool.peer_shape[3] == k
              and not symm_mem_pool.gather_bitmatrix)
    if direct:
        vals_loc, indx_loc = symm_mem_pool.route_vals, symm_mem_pool.route_indx
    _lib.check(lib.moe_topk_fwd(_lib.ptr(x), _lib.dtype_code(x.dtype), T, E, k, int(bool(apply_softmax)), x.stride(0),
                                _lib.ptr(vals_loc), vals_loc.stride(0), _lib.ptr(indx_loc), indx_loc.stride(0),
                                _lib.ptr(bm_loc), bm.stride(0), bm.stride(1), _lib.ptr(n_rows_dev), int(use_provided),
                                _lib.stream()), "moe_topk_fwd")
    if all_gather and world > 1:
        symm_mem_pool.all_gather_routing(y_vals, None if use_provided else y_indx_full, bm_store, T, rank, published=direct)
    shape0 = (n_rows if n_rows is not None else T)
    if all_gather and world > 1:
        shape0 = T_out
    bitmatrix = wrap_torch_tensor(bm, dtype=BIT, shape=[shape0, E], shape_max=[T_out, None])
    return y_vals, y_indx_full[:T_out], bitmatrix


def topk(x: Union[Tensor, torch.Tensor], k: int, apply_softmax: bool = True, dim: int = 1,
         y_indx: Optional[torch.Tensor] = None, n_rows: Optional[int] = None, all_gather: bool = False,
         symm_mem_pool=None):
    """Top-k values and indices of each row of `x` ([n_tokens, n_expts]); returns a SparseMatrix whose
    `mask_metadata` holds the expert histogram and the expert-major sort (triton_kernels/topk.py:106-141)."""
    y_vals, y_indx, bitmatrix = topk_forward(x, k, apply_softmax, dim, y_indx, n_rows, all_gather, symm_mem_pool)
    return SparseMatrix(vals=y_vals, indx=y_indx, mask=bitmatrix)
