"""Standalone SwiGLU and the k-way combine (reduce) on the GPU against the oracle and the reference fixture."""
import pytest
import torch

import oracle
import triton_b200 as tb
from triton_b200.swiglu import PrecisionConfig as SwigluPC

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M, N", [(1311, 4352), (7, 34), (256, 2880)])
@pytest.mark.parametrize("limit", [1e-2, 10, None])
def test_swiglu(M, N, limit, device):
    # reference tests/test_swiglu.py:23-32
    torch.manual_seed(0)
    x = torch.randn(M, N, device=device).bfloat16()
    y = tb.swiglu(x, 0.5, SwigluPC(limit))
    ref = oracle.swiglu_oracle(x.cpu().float(), 0.5, limit).bfloat16()
    oracle.assert_close_oracle(ref, y.cpu())


def test_swiglu_and_reduce_against_reference_fixture(golden, device):
    g = golden("gemm_small")
    act = tb.swiglu(g["y_plain"].to(device), g["alpha"], SwigluPC(g["limit"]))
    oracle.assert_close_oracle(g["act"], act.cpu())
    red, _ = tb.reduce(g["yk"].to(device), 1, mask=g["mask"].to(device))
    torch.testing.assert_close(red.cpu().float(), g["red"].float(), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("shape", [(25, 2, 48), (4096, 4, 2880), (3, 5, 7)])
@pytest.mark.parametrize("dim", [0, 1, 2])
@pytest.mark.parametrize("mask_mode", ["none", "row", "full"])
def test_reduce(shape, dim, mask_mode, device):
    # reference tests/test_reduce.py:41-121 (tolerance 1e-3)
    if shape[0] > 1000 and dim != 1:
        pytest.skip("large case is the combine only")
    torch.manual_seed(0)
    x = torch.randn(shape, device=device).bfloat16()
    mask = None
    if mask_mode == "row":
        mshape = list(shape)
        mshape[2] = 1
        mask = (torch.rand(mshape, device=device) > 0.3).expand(shape)
    elif mask_mode == "full":
        mask = (torch.rand(shape, device=device) > 0.3).to(torch.int32)
    scale = torch.rand(shape[0], shape[1], 1, device=device) if mask_mode != "full" else None
    y, _ = tb.reduce(x, dim, mask=mask, scale=scale)
    ref = oracle.reduce_oracle(x.cpu(), dim, None if mask is None else mask.cpu(), None if scale is None else scale.cpu())
    torch.testing.assert_close(y.cpu().float(), ref.float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("n_out, d", [(500, 96), (5000, 2880), (40000, 64), (700001, 32)])
def test_gather_rows_over_peer_buffers(n_out, d, device):
    """moe_gather_rows_peers with three buffers on one device standing in for three ranks: -1 writes zeros, -2 leaves
    the row untouched.  The sizes walk the kernel's rows-per-warp batches from 1 (few rows) to 32 (many)."""
    import ctypes
    from triton_b200 import _lib
    torch.manual_seed(0)
    rows_per_peer = 37
    bufs = [torch.randn(rows_per_peer, d, device=device).bfloat16() for _ in range(3)]
    allrows = torch.cat(bufs)
    idx = torch.randint(0, 3 * rows_per_peer, (n_out,), device=device, dtype=torch.int32)
    idx[::7] = -1
    idx[3::11] = -2
    idx[torch.rand(n_out, device=device) < 0.6] = -2          # most rows belong to other ranks
    out = torch.full((n_out, d), 7.0, device=device).bfloat16()
    lib = _lib.load()
    ptrs = (ctypes.c_void_p * 3)(*[b.data_ptr() for b in bufs])
    _lib.check(lib.moe_gather_rows_peers(ptrs, 3, rows_per_peer, d * 2, _lib.ptr(idx), n_out, d * 2, _lib.ptr(out), d * 2,
                                         _lib.stream()), "moe_gather_rows_peers")
    want = allrows[idx.long().clamp_min(0)]
    want[idx == -1] = 0
    want[idx == -2] = 7.0
    assert torch.equal(out, want)


def test_allgather_over_peer_buffers(device):
    import ctypes
    from triton_b200 import _lib
    torch.manual_seed(0)
    slices = [torch.randint(-1000, 1000, (37, 4), dtype=torch.int16, device=device) for _ in range(3)]
    out = torch.zeros((3 * 37, 4), dtype=torch.int16, device=device)
    lib = _lib.load()
    ptrs = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in slices])
    _lib.check(lib.moe_allgather_peers(ptrs, 3, 37 * 4 * 2, _lib.ptr(out), _lib.stream()), "moe_allgather_peers")
    assert torch.equal(out, torch.cat(slices))


def test_peer_barrier_counts_epochs_and_its_wait_is_bounded(device):
    """One rank alone passes its own barrier and counts epochs; a barrier whose second rank never arrives gives up
    after its time limit, reports status 901 and leaves the device usable."""
    import ctypes
    import time
    from triton_b200 import _lib
    lib = _lib.load()
    sig = torch.zeros(16, dtype=torch.int32, device=device)
    epoch = torch.zeros(1, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    one = (ctypes.c_void_p * 1)(sig.data_ptr())
    for _ in range(3):
        _lib.check(lib.moe_peer_barrier(one, 1, 0, _lib.ptr(epoch), _lib.ptr(status), _lib.stream()), "moe_peer_barrier")
    torch.cuda.synchronize()
    assert int(epoch.item()) == 3 and int(sig[0].item()) == 3 and int(status.item()) == 0
    # two ranks' signal buffers, but only rank 0 ever calls: its wait for rank 1's word runs out
    sig0, sig1 = torch.zeros(16, dtype=torch.int32, device=device), torch.zeros(16, dtype=torch.int32, device=device)
    epoch.zero_()
    two = (ctypes.c_void_p * 2)(sig0.data_ptr(), sig1.data_ptr())
    t0 = time.time()
    _lib.check(lib.moe_peer_barrier(two, 2, 0, _lib.ptr(epoch), _lib.ptr(status), _lib.stream()), "moe_peer_barrier")
    torch.cuda.synchronize()
    assert 1.5 < time.time() - t0 < 10.0
    assert int(status.item()) == 901
    assert int(sig1[0].item()) == 1 and int(sig0[0].item()) == 1          # rank 0's word arrived on both "ranks"
    # the same code through the layer's status word is reported as a peer-barrier time-out, not as a GEMM pipeline wait
    from triton_b200.matmul import _status_word, matmul_check_status
    _status_word(torch.device(device)).fill_(901)
    with pytest.raises(RuntimeError, match="peer barrier"):
        matmul_check_status(device)
    matmul_check_status(device)                                            # the word was cleared
    assert float((torch.ones(8, device=device) * 2).sum().item()) == 16.0     # the context is still healthy


def test_gather_reduce_over_peer_buffers(device):
    """k-way combine whose rows live in three buffers (one device standing in for three ranks); -1 entries are skipped."""
    import ctypes
    from triton_b200 import _lib
    torch.manual_seed(0)
    rows_per_peer, d, T, k = 50, 2880, 40, 4
    bufs = [torch.randn(rows_per_peer, d, device=device).bfloat16() for _ in range(3)]
    allrows = torch.cat(bufs)
    idx = torch.randint(0, 3 * rows_per_peer, (T, k), device=device, dtype=torch.int32)
    idx[::5, 1] = -1
    idx[1::7, 3] = -1                                 # dropped entries whose neighbours live on the last buffer
    out = torch.empty((T, d), device=device, dtype=torch.bfloat16)
    lib = _lib.load()
    ptrs = (ctypes.c_void_p * 3)(*[b.data_ptr() for b in bufs])
    _lib.check(lib.moe_gather_reduce_rows_peers(ptrs, 3, rows_per_peer, d, _lib.ptr(idx), T, k, d, _lib.ptr(out), d,
                                                _lib.stream()), "moe_gather_reduce_rows_peers")
    picked = allrows[idx.long().clamp_min(0)].float() * (idx >= 0).unsqueeze(-1)
    want = picked[:, 0]
    for j in range(1, k):
        want = want + picked[:, j]                    # same order of fp32 additions as the kernel
    assert torch.equal(out, want.bfloat16())
