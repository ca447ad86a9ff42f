"""Expert histogram and the stable expert-major sort of the routed (token, slot) entries
(triton_kernels/tensor_details/bitmatrix.py:8-25, 110-150)."""
from dataclasses import dataclass

import torch

from .. import _lib


@dataclass
class BitmatrixMetadata:
    """`col_sum[e]`: entries routed to expert e.  `col_sorted_indx[p]`: flat index (token * k + slot) of the
    p-th entry in expert-major, stable order.  `row_sorted_indx[i]`: p for flat index i (the inverse).
    Dropped entries are skipped; both index arrays are padded with -1."""
    col_sum: torch.Tensor
    col_sorted_indx: torch.Tensor
    row_sorted_indx: torch.Tensor


def make_bitmatrix_metadata(nonzero_indx, bitmatrix):
    """nonzero_indx: int16 [n_tokens_max, k] expert ids (the top-k output); bitmatrix: the BIT Tensor whose
    `shape[0]` may be a device scalar bounding the valid rows and whose `shape[1]` is the expert count."""
    assert nonzero_indx.ndim == 2
    lib = _lib.load()
    T, k = nonzero_indx.shape
    E = int(bitmatrix.shape[1])
    n_rows = bitmatrix.shape[0]
    n_rows_dev = n_rows if isinstance(n_rows, torch.Tensor) else None
    if n_rows_dev is None and int(n_rows) < T:
        n_rows_dev = torch.tensor([int(n_rows)], dtype=torch.int32, device=nonzero_indx.device)
    if n_rows_dev is not None:
        n_rows_dev = n_rows_dev.to(torch.int32)
    dev = nonzero_indx.device
    if nonzero_indx.dtype != torch.int16:
        nonzero_indx = nonzero_indx.to(torch.int16)
    if nonzero_indx.stride(1) != 1:
        nonzero_indx = nonzero_indx.contiguous()
    col_sum = torch.empty(E, dtype=torch.int32, device=dev)
    combined = torch.empty(2 * T * k, dtype=torch.int32, device=dev)
    col_sorted, row_sorted = combined[: T * k], combined[T * k:]
    ws_bytes = lib.moe_bitmatrix_metadata_workspace(T, E, k)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    _lib.check(lib.moe_bitmatrix_metadata(_lib.ptr(nonzero_indx), nonzero_indx.stride(0), T, E, k, _lib.ptr(n_rows_dev),
                                          _lib.ptr(col_sum), _lib.ptr(col_sorted), _lib.ptr(row_sorted), _lib.ptr(ws),
                                          ws_bytes, _lib.stream()), "moe_bitmatrix_metadata")
    return BitmatrixMetadata(col_sum=col_sum, col_sorted_indx=col_sorted, row_sorted_indx=row_sorted)
