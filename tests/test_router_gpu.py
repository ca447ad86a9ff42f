"""Router product fused with the top-k selection (`moe_router_topk`) against the CPU oracle of the reference's
`topk(matmul(x, wg, bg), k)` (bench/bench_mlp.py:70, topk.py:144-185).

Two comparisons, because the fp32 sums of a tensor-core product differ from the oracle's in their last bits and a
selection can legitimately flip where two logits are that close: (1) the logits the kernel selected from against the
oracle's logits, within a tolerance; (2) selection, softmax and bitmatrix against the oracle's `topk` run ON those
logits, exactly (indices, bitmatrix) and to 2e-6 (values)."""
import pytest
import torch

import oracle
import triton_b200 as tb

pytestmark = pytest.mark.gpu

CASES = [
    # T, K, E, k
    (1, 2880, 128, 4),          # one token: K cut into slices over the SMs
    (64, 2880, 128, 4),
    (130, 64, 256, 16),         # one k step, two token blocks, the widest MMA
    (200, 512, 32, 2),
    (300, 320, 48, 8),          # experts not a multiple of 32
    (1000, 2880, 128, 4),
    (4096, 2880, 128, 1),
    (16384, 2880, 128, 4),      # the stand-alone routing configuration: one slice per token block
]


def make(T, K, E, seed, bias):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, K, generator=g).bfloat16()
    wg = (torch.randn(K, E, generator=g) / K ** 0.5).bfloat16()
    bg = torch.randn(E, generator=g) if bias else None
    return x, wg, bg


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("logits_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bias", [False, True])
def test_router_topk_against_oracle(case, logits_dtype, bias, device):
    T, K, E, k = case
    if T >= 4096 and not bias:
        pytest.skip("large cases run once")
    x, wg, bg = make(T, K, E, T + K + E, bias)
    wg_dev = tb.prepare_router_weight(wg.to(device))
    sp, logits = tb.router_topk(x.to(device), wg_dev, None if bg is None else bg.to(device), k, logits_dtype=logits_dtype,
                                return_logits=True)
    tb.matmul_check_status()
    ref_logits, _, _, _ = oracle.router_topk_oracle(x, wg, bg, k, True, logits_dtype)
    got = logits.cpu()
    if logits_dtype == torch.float32:
        assert (got - ref_logits).abs().max().item() < 2e-4        # fp32 sums over K in another order
    else:
        # equal after the rounding, except where the fp32 sum sat at a rounding boundary: then one bf16 step apart
        diff = (got - ref_logits.float()).abs()
        step = (ref_logits.float().abs() * 2.0 ** -7).clamp_min(1e-5)         # logits near zero: the sums' absolute error
        assert (diff <= step).all()
        assert (diff > 0).float().mean().item() < 5e-3
    # the selection, on the logits the kernel saw
    vals, indx, bm = oracle.topk_oracle(got.to(logits_dtype), k, True)
    assert sp.vals.dtype == logits_dtype and sp.indx.dtype == torch.int16
    assert torch.equal(sp.indx.cpu().int(), indx)
    assert torch.equal(sp.mask.storage.data.cpu()[:T], bm)
    tol = 2e-6 if logits_dtype == torch.float32 else 2.0 ** -8
    assert (sp.vals.cpu().float() - vals.float()).abs().max().item() <= tol
    # the metadata built from the fused selection is what the stand-alone routing gives for the same logits
    ref_sp = tb.topk(got.to(logits_dtype).to(device), k)
    assert torch.equal(sp.mask_metadata.col_sum, ref_sp.mask_metadata.col_sum)
    assert torch.equal(sp.mask_metadata.col_sorted_indx, ref_sp.mask_metadata.col_sorted_indx)


def test_router_topk_equal_logits_go_to_the_smaller_expert(device):
    """Identical expert columns give identical logits: the selection must take the smaller indices, in order."""
    T, K, E, k = 70, 256, 64, 4
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, K, generator=g).bfloat16()
    col = (torch.randn(K, 1, generator=g) / 16).bfloat16()
    wg = col.repeat(1, E).contiguous()
    sp = tb.router_topk(x.to(device), wg.to(device), None, k, apply_softmax=False, logits_dtype=torch.float32)
    tb.matmul_check_status()
    assert torch.equal(sp.indx.cpu().int(), torch.arange(k, dtype=torch.int32).repeat(T, 1))
    v = sp.vals.cpu()
    assert torch.equal(v, v[:, :1].repeat(1, k))


def test_router_topk_falls_back_for_other_shapes(device):
    """More than 256 experts: the two steps run apart and give the same kind of result."""
    T, K, E, k = 50, 128, 320, 4
    x, wg, bg = make(T, K, E, 3, True)
    sp = tb.router_topk(x.to(device), wg.to(device), bg.to(device), k, logits_dtype=torch.float32)
    logits, vals, indx, bm = oracle.router_topk_oracle(x, wg, bg, k, True, torch.float32)
    assert sp.indx.shape == (T, k)
    agree = (sp.indx.cpu().int() == indx).all(dim=1).float().mean().item()
    assert agree > 0.95


@pytest.mark.parametrize("name", ["router_T50_E32_k4", "router_T9_E128_k2"])
def test_router_topk_against_reference_fixture(golden, name, device):
    """Fixtures recorded from the reference's own `matmul_torch` + `topk_torch`."""
    g = golden(name)
    k = int(g["k"])
    sp, logits = tb.router_topk(g["x"].to(device), g["wg"].to(device), g["bg"].to(device), k, return_logits=True)
    tb.matmul_check_status()
    ref = g["logits"].float()
    diff = (logits.cpu() - ref).abs()
    assert (diff <= (ref.abs() * 2.0 ** -7).clamp_min(1e-5)).all()
    same = diff.max(dim=1).values == 0           # rows whose logits came out bit-identical must select identically
    assert same.float().mean().item() > 0.9
    assert torch.equal(sp.indx.cpu().int()[same], g["indx"].int()[same])
    assert torch.equal(sp.mask.storage.data.cpu()[: ref.shape[0]][same], g["bitmatrix"][same])
    assert (sp.vals.cpu().float()[same] - g["vals"].float()[same]).abs().max().item() <= 2.0 ** -8
