"""Routing on the GPU (top-k + bitmatrix, histogram + expert-major sort, ragged metadata, remap),
bit-exact against the reference fixtures and the CPU oracle."""
import pytest
import torch

import oracle
from triton_b200 import (make_bitmatrix_metadata, make_ragged_tensor_metadata, remap_ragged_tensor_metadata, routing,
                         topk)
from triton_b200.tensor import BIT, RaggedTensorMetadata, wrap_torch_tensor

pytestmark = pytest.mark.gpu


def check_topk(logits_cpu, k, softmax, device, n_rows=None):
    sp = topk(logits_cpu.to(device), k, apply_softmax=softmax, n_rows=n_rows)
    vals, indx, bm = oracle.topk_oracle(logits_cpu, k, softmax, n_rows=n_rows)
    nr = logits_cpu.shape[0] if n_rows is None else n_rows
    assert sp.indx.dtype == torch.int16
    assert torch.equal(sp.indx[:nr].cpu().int(), indx[:nr])
    T, E = logits_cpu.shape
    data = sp.mask.storage.data
    assert data.shape == (T, (E + 31) // 32) and data.stride() == (1, (T + 31) // 32 * 32)
    assert torch.equal(data[:nr].cpu(), bm[:nr])
    if softmax:
        torch.testing.assert_close(sp.vals[:nr].cpu().float(), vals[:nr].float(), atol=2e-6, rtol=2e-5)
    else:
        assert torch.equal(sp.vals[:nr].cpu(), vals[:nr])
    return sp, indx


@pytest.mark.parametrize("name", ["topk_T7_E13_k4", "topk_T256_E128_k4", "topk_T300_E200_k8", "topk_T33_E32_k2"])
def test_against_reference_fixture(golden, name, device):
    g = golden(name)
    sp = topk(g["logits"].to(device), g["k"], apply_softmax=bool(g["softmax"]))
    assert torch.equal(sp.indx.cpu().int(), g["indx"].int())
    assert torch.equal(sp.mask.storage.data.cpu(), g["bitmatrix"])
    torch.testing.assert_close(sp.vals.cpu(), g["vals"], atol=2e-6, rtol=2e-5)
    md = sp.mask_metadata
    assert torch.equal(md.col_sum.cpu(), g["col_sum"].int())
    assert torch.equal(md.col_sorted_indx.cpu(), g["col_sorted"])
    assert torch.equal(md.row_sorted_indx.cpu(), g["row_sorted"])


@pytest.mark.parametrize("T", [1, 7, 256, 300])
@pytest.mark.parametrize("E", [13, 32, 128, 200])
@pytest.mark.parametrize("softmax", [True, False])
def test_topk_grid(T, E, softmax, device):
    # reference tests/test_topk.py:11-29 (k = 8)
    torch.manual_seed(T * 1000 + E)
    logits = torch.randn(T, E)
    logits[:, min(3, E - 1)] = logits[:, 0]              # ties
    check_topk(logits, 8, softmax, device)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_topk_low_precision_logits(dt, device):
    torch.manual_seed(1)
    logits = torch.randn(65, 64).to(dt)                  # many exact ties after rounding
    sp = topk(logits.to(device), 4, apply_softmax=False)
    vals, indx, bm = oracle.topk_oracle(logits, 4, False)
    assert torch.equal(sp.indx.cpu().int(), indx) and torch.equal(sp.vals.cpu(), vals)


def test_topk_n_rows_and_provided_indx(device):
    torch.manual_seed(2)
    logits = torch.randn(100, 40)
    sp, indx = check_topk(logits, 4, True, device, n_rows=61)
    md = sp.mask_metadata
    cs, col, row = oracle.bitmatrix_metadata_oracle(indx, 40)
    assert torch.equal(md.col_sum.cpu(), cs)
    assert torch.equal(md.col_sorted_indx.cpu(), col) and torch.equal(md.row_sorted_indx.cpu(), row)
    yi = torch.stack([torch.randperm(40)[:4] for _ in range(100)]).to(torch.int16)
    sp2 = topk(logits.to(device), 4, apply_softmax=True, y_indx=yi.to(device))
    vals, indx2, bm = oracle.topk_oracle(logits, 4, True, y_indx=yi)
    assert torch.equal(sp2.indx.cpu(), yi) and torch.equal(sp2.mask.storage.data.cpu(), bm)
    torch.testing.assert_close(sp2.vals.cpu(), vals, atol=2e-6, rtol=2e-5)


@pytest.mark.parametrize("T", [7, 256, 17111])
@pytest.mark.parametrize("E", [13, 32, 128, 811])
@pytest.mark.parametrize("k", [1, 4, 8])
def test_bitmatrix_metadata_grid(T, E, k, device):
    # reference tests/test_tensor.py:280-302
    torch.manual_seed(T + E + k)
    indx = torch.stack([torch.randperm(E)[:k] for _ in range(min(T, 512))])
    indx = indx.repeat((T + indx.shape[0] - 1) // indx.shape[0], 1)[:T]
    indx = indx[torch.randperm(T)].to(torch.int16)
    bm = wrap_torch_tensor(torch.empty((T, (E + 31) // 32), dtype=torch.int32, device=device), dtype=BIT, shape=[T, E])
    md = make_bitmatrix_metadata(indx.to(device), bm)
    cs, col, row = oracle.bitmatrix_metadata_oracle(indx.int(), E)
    assert torch.equal(md.col_sum.cpu(), cs)
    assert torch.equal(md.row_sorted_indx.cpu(), row)
    assert torch.equal(md.col_sorted_indx.cpu(), col)


@pytest.mark.parametrize("n_slices", [1, 7, 33, 911, 1025])
def test_ragged_metadata_and_remap(n_slices, device):
    # reference tests/test_tensor.py:243-277
    torch.manual_seed(n_slices)
    sizes = torch.randint(0, 300, (n_slices,), dtype=torch.int32)
    sizes[torch.randint(0, n_slices, (1,))] = 0
    n_rows = int(sizes.sum()) + 100
    md = make_ragged_tensor_metadata(sizes.to(device), n_rows)
    so, bo, bs = oracle.ragged_metadata_oracle(sizes, n_rows)
    assert torch.equal(md.slice_offs.cpu(), so)
    assert torch.equal(md.block_offs_data.cpu(), bo)
    assert torch.equal(md.block_schedule_data.cpu(), bs)
    assert md.block_schedule_data.shape[1] == RaggedTensorMetadata.max_n_blocks(n_slices, n_rows)
    smap = torch.full((n_slices,), -1, dtype=torch.int32)
    keep = torch.randperm(n_slices)[: max(1, n_slices - 5)].sort().values
    smap[keep] = torch.randperm(keep.numel()).int()
    r = remap_ragged_tensor_metadata(md, smap.to(device))
    ro = oracle.remap_ragged_metadata_oracle(sizes, so, bo, bs, smap)
    assert torch.equal(r.slice_sizes.cpu(), ro[0]) and torch.equal(r.slice_offs.cpu(), ro[1])
    assert torch.equal(r.block_offs_data.cpu(), ro[2]) and torch.equal(r.block_schedule_data.cpu(), ro[3])


@pytest.mark.parametrize("name", ["ragged_E1", "ragged_E7", "ragged_E33", "ragged_E130"])
def test_ragged_against_reference_fixture(golden, name, device):
    g = golden(name)
    md = make_ragged_tensor_metadata(g["slice_sizes"].to(device), g["n_rows"])
    assert torch.equal(md.slice_offs.cpu(), g["slice_offs"])
    assert torch.equal(md.block_offs_data.cpu(), g["block_offs"])
    assert torch.equal(md.block_schedule_data.cpu(), g["block_schedule"])
    r = remap_ragged_tensor_metadata(md, g["slice_map"].to(device))
    assert torch.equal(r.slice_sizes.cpu(), g["r_slice_sizes"]) and torch.equal(r.slice_offs.cpu(), g["r_slice_offs"])
    assert torch.equal(r.block_offs_data.cpu(), g["r_block_offs"])
    assert torch.equal(r.block_schedule_data.cpu(), g["r_block_schedule"])


def test_routing_full_size(device):
    """fp32 logits [16384, 128], top-4 + softmax: indices, histogram and both index arrays equal the oracle's;
    the two index arrays are inverse permutations and the sort is expert-major and stable."""
    torch.manual_seed(0)
    logits = torch.randn(16384, 128)
    ragged, gather_idx, scatter_idx, sp = routing(logits.to(device), 4)
    vals, indx, bm = oracle.topk_oracle(logits, 4, True)
    assert torch.equal(sp.indx.cpu().int(), indx) and torch.equal(sp.mask.storage.data.cpu(), bm)
    cs, col, row = oracle.bitmatrix_metadata_oracle(indx, 128)
    md = sp.mask_metadata
    assert torch.equal(md.col_sum.cpu(), cs) and torch.equal(md.col_sorted_indx.cpu(), col)
    assert torch.equal(md.row_sorted_indx.cpu(), row)
    assert torch.equal(md.row_sorted_indx[md.col_sorted_indx.long()].cpu(), torch.arange(65536, dtype=torch.int32))
    e_sorted = sp.indx.reshape(-1)[md.col_sorted_indx.long()].int()
    assert (e_sorted[1:] >= e_sorted[:-1]).all()
    same = e_sorted[1:] == e_sorted[:-1]
    assert (md.col_sorted_indx[1:][same] > md.col_sorted_indx[:-1][same]).all()
    so, bo, bs = oracle.ragged_metadata_oracle(cs, 65536)
    assert torch.equal(ragged.slice_offs.cpu(), so) and torch.equal(ragged.block_offs_data.cpu(), bo)
    assert torch.equal(ragged.block_schedule_data.cpu(), bs)
    assert torch.equal(gather_idx.cpu(), col // 4) and torch.equal(scatter_idx.cpu(), col)


@pytest.mark.parametrize("T, E, k", [(1, 128, 4), (7, 13, 2), (255, 32, 4), (256, 128, 4), (257, 200, 8), (4099, 256, 4),
                                     (16384, 128, 4), (129, 48, 3), (1000, 128, 6), (300, 64, 16), (2500, 96, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_route_equals_separate_entry_points(T, E, k, dtype, device, monkeypatch):
    """`route` (three launches: top-k + histogram, scan + ragged metadata, rank) returns exactly what the five-launch
    composition topk -> make_bitmatrix_metadata -> make_ragged_tensor_metadata returns, and what the oracle computes."""
    import importlib
    routing_mod = importlib.import_module("triton_b200.routing")      # (the package exports a function of the same name)
    route = routing_mod.route
    monkeypatch.setattr(routing_mod, "FUSED_MAX_TOKENS", 1 << 30)      # the fused form at every size
    torch.manual_seed(T * 131 + E)
    logits = torch.randn(T, E, device=device).to(dtype)
    if T > 2:
        logits[1] = logits[0]                      # equal rows and ties inside a row
        logits[2, : E // 2] = logits[2, E // 2: 2 * (E // 2)]
    ragged, sp = route(logits, k)
    sp2 = topk(logits, k)
    md, md2 = sp.mask_metadata, sp2.mask_metadata
    rg2 = make_ragged_tensor_metadata(md2.col_sum, T * k)
    assert torch.equal(sp.indx, sp2.indx) and torch.equal(sp.vals, sp2.vals)
    assert torch.equal(sp.mask.storage.data[:T], sp2.mask.storage.data[:T])
    assert torch.equal(md.col_sum, md2.col_sum) and torch.equal(md.col_sorted_indx, md2.col_sorted_indx)
    assert torch.equal(md.row_sorted_indx, md2.row_sorted_indx)
    assert torch.equal(ragged.slice_offs, rg2.slice_offs) and torch.equal(ragged.block_offs_data, rg2.block_offs_data)
    assert torch.equal(ragged.block_schedule_data, rg2.block_schedule_data)
    # and the oracle
    vals_o, indx_o, _ = oracle.topk_oracle(logits.cpu(), k, apply_softmax=True)
    assert torch.equal(sp.indx.cpu().long(), indx_o.long())
    col_sum_o, col_sorted_o, row_sorted_o = oracle.bitmatrix_metadata_oracle(indx_o, E)
    assert torch.equal(md.col_sum.cpu().long(), col_sum_o.long())
    assert torch.equal(md.col_sorted_indx.cpu().long(), col_sorted_o.long())
    assert torch.equal(md.row_sorted_indx.cpu().long(), row_sorted_o.long())
