"""moe_bitmatrix_metadata_noalloc: the histogram + expert-major sort with the library's built-in scratch, for
callers that cannot allocate a workspace (all device memory already in their own pools, or no cudaMalloc allowed
where they call from).  Called through the C ABI, twice in a row with different inputs, and compared with
moe_bitmatrix_metadata given a caller-allocated workspace: the integer outputs must be identical.

This file sorts last on purpose, so that a run that stops at the first failure has already run every other test."""
import pytest
import torch

from triton_b200 import _lib

pytestmark = pytest.mark.gpu


def _inputs(T, E, k, seed, device):
    g = torch.Generator().manual_seed(seed)
    rows = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(min(T, 256))])
    indx = rows.repeat((T + rows.shape[0] - 1) // rows.shape[0], 1)[:T]
    indx = indx[torch.randperm(T, generator=g)].to(torch.int16).contiguous()
    return indx.to(device)


def _outputs(T, E, k, device):
    # poisoned, so that an entry the kernels fail to write shows up
    return (torch.full((E,), -7, dtype=torch.int32, device=device),
            torch.full((T * k,), -7, dtype=torch.int32, device=device),
            torch.full((T * k,), -7, dtype=torch.int32, device=device))


def _with_workspace(lib, indx, T, E, k, n_rows, device):
    cs, col, row = _outputs(T, E, k, device)
    nbytes = lib.moe_bitmatrix_metadata_workspace(T, E, k)
    ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=device)
    _lib.check(lib.moe_bitmatrix_metadata(_lib.ptr(indx), indx.stride(0), T, E, k, _lib.ptr(n_rows), _lib.ptr(cs),
                                          _lib.ptr(col), _lib.ptr(row), _lib.ptr(ws), nbytes, _lib.stream()))
    return cs, col, row


def _no_alloc(lib, indx, T, E, k, n_rows, device):
    cs, col, row = _outputs(T, E, k, device)
    _lib.check(lib.moe_bitmatrix_metadata_noalloc(_lib.ptr(indx), indx.stride(0), T, E, k, _lib.ptr(n_rows), _lib.ptr(cs),
                                                  _lib.ptr(col), _lib.ptr(row), _lib.stream()))
    return cs, col, row


def test_no_alloc_entry_point_matches_workspace_entry_point(device):
    lib = _lib.load()
    assert lib.moe_bitmatrix_metadata_noalloc_capacity() == 1 << 20
    # two calls in a row that share the built-in scratch: a large problem, then a smaller one with a different
    # expert count and some rows masked off, so stale contents of the first call would be noticed
    cases = [(16384, 128, 4, None, 1), (1000, 37, 2, 777, 2)]
    for T, E, k, n_rows_val, seed in cases:
        indx = _inputs(T, E, k, seed, device)
        n_rows = None if n_rows_val is None else torch.tensor([n_rows_val], dtype=torch.int32, device=device)
        ref = _with_workspace(lib, indx, T, E, k, n_rows, device)
        got = _no_alloc(lib, indx, T, E, k, n_rows, device)
        torch.cuda.synchronize()
        for r, g in zip(ref, got):
            assert torch.equal(r, g)                      # integer outputs: identical, no tolerance
        assert int(ref[0].sum()) == (T if n_rows_val is None else n_rows_val) * k


def test_no_alloc_entry_point_rejects_oversized_problems(device):
    lib = _lib.load()
    T, E, k = 1 << 20, 128, 4                            # needs 4096 * 128 + 128 ints = 2 MiB > 1 MiB
    st = lib.moe_bitmatrix_metadata_noalloc(None, k, T, E, k, None, None, None, None, None)
    assert st == 1
    msg = lib.moe_last_error().decode()
    assert "built-in" in msg and "moe_bitmatrix_metadata" in msg
