"""The block-scaled grouped GEMM (tcgen05.mma.kind::mxf8f6f4: MXFP4 weights straight into the MMA) on the GPU against
the CPU oracle: e4m3 and MXFP8 activations (the reference's `a_mx_scale` mode, tests/test_matmul.py:282-285), and bf16
activations split inside the library into two e4m3 terms, or (small token blocks) into four e2m1 terms for
tcgen05.mma.kind::mxf4."""
import pytest
import torch

import oracle
import triton_b200 as tb
from triton_b200.tensor import FP4, convert_layout, wrap_torch_tensor
from triton_b200.tensor_details.layout import B200BlockScaledScaleLayout, B200BlockScaledValueLayout

pytestmark = pytest.mark.gpu

MAXTOL_MX4 = 3e-2          # the reference's bound for MXFP4 weights (tests/test_matmul.py:649-650)


def quantised_weights(E, K, N, g, unit_scales=False, w_std=0.02):
    w = (torch.randn(E, K, N, generator=g) * w_std).bfloat16()
    wq, ws = oracle.downcast_to_mxfp_oracle(w, 1)
    if unit_scales:
        ws = torch.full_like(ws, 127)
    # K contiguous, as downcast_to_mxfp(axis=1) returns it
    wq = wq.contiguous().transpose(1, 2).contiguous().transpose(1, 2)
    ws = ws.contiguous().transpose(1, 2).contiguous().transpose(1, 2)
    return wq, ws, oracle.dequant_weight_oracle(wq, ws)


def to_block_scaled(wq, ws, device):
    tq = convert_layout(wrap_torch_tensor(wq.to(device), dtype=FP4), B200BlockScaledValueLayout())
    ts = convert_layout(wrap_torch_tensor(ws.to(device)), B200BlockScaledScaleLayout())
    return tq, ts


def test_block_scaled_layout_round_trip(device):
    g = torch.Generator().manual_seed(3)
    for E, K, N in [(2, 96, 40), (3, 2880, 200), (1, 128, 128)]:
        wq = torch.randint(0, 256, (E, N, K // 2), generator=g, dtype=torch.uint8).transpose(1, 2)   # [E, K/2, N], K contiguous
        ws = torch.randint(0, 255, (E, N, K // 32), generator=g, dtype=torch.uint8).transpose(1, 2)
        tq, ts = to_block_scaled(wq, ws, device)
        KT, NB = (K + 127) // 128, (N + 127) // 128
        assert tq.storage.data.numel() == E * KT * NB * 128 * 64 and ts.storage.data.numel() == E * KT * NB * 512
        # spot-check the documented positions on the host
        v = tq.storage.data.cpu().view(E, KT, NB, 128, 64)
        s = ts.storage.data.cpu().view(E, KT, NB, 32, 4, 4)
        for (e, n, k) in [(0, 0, 0), (E - 1, N - 1, K - 2), (0, min(N - 1, 33), min(K - 2, 70))]:
            assert int(v[e, k // 128, n // 128, n % 128, (k % 128) // 2]) == int(wq[e, k // 2, n])
            assert int(s[e, k // 128, n // 128, (n % 128) % 32, (n % 128) // 32, (k % 128) // 32]) == int(ws[e, k // 32, n])
        from triton_b200.tensor_details.layout import StridedLayout
        back_q = convert_layout(tq, StridedLayout(major_dim=-2))
        back_s = convert_layout(ts, StridedLayout(major_dim=-2))
        assert torch.equal(back_q.storage.data.cpu(), wq) and torch.equal(back_s.storage.data.cpu(), ws)


def run_mx(x, wq, ws, sizes, device, *, a_scale=None, bias=None, gather=None, scatter=None, gammas=None, betas=None,
           act=None, out_dtype=torch.bfloat16, block_m=None, block_n=None, kernel=None):
    dev = lambda t: None if t is None else t.to(device)
    tq, ts = to_block_scaled(wq, ws, device)
    M = int(sizes.sum())
    md = tb.make_ragged_tensor_metadata(dev(sizes), M)
    pc = tb.PrecisionConfig(b_mx_scale=ts, b_microblock_size=32, a_mx_scale=dev(a_scale), out_dtype=out_dtype)
    fa = None
    if act:
        fa = tb.FusedActivation(tb.FnSpecs("swiglu", tb.swiglu_fn, ("alpha", "limit"), reduction_n=2), act)
    cons = {}
    if block_m:
        cons["block_m"] = block_m
    if block_n:
        cons["block_n"] = block_n
    if kernel:
        cons["kernel"] = kernel
    with tb.scoped_opt_flags_constraints(cons):
        y = tb.matmul(dev(x), tq, dev(bias), md, None, dev(gather), dev(scatter), pc, betas=dev(betas), gammas=dev(gammas),
                      fused_activation=fa)
    tb.matmul_check_status()
    return y.cpu()


def dequant_act(x8, a_scale):
    xf = x8.float()
    if a_scale is not None:
        xf = (xf.view(x8.shape[0], -1, 32) * torch.exp2(a_scale.float() - 127.0)[:, :, None]).reshape(x8.shape)
    return xf


@pytest.mark.parametrize("stage", ["unit-scales", "weight-scales", "act-scales"])
@pytest.mark.parametrize("block_n", [128, 384])
def test_block_scaled_dense_fp8_exact_products(stage, block_n, device):
    """One expert, e4m3 activations: every product is exact in the tensor core and the sum is fp32, so the result
    must match the fp32 oracle closely.  The three stages separate the value path (unit scales), the weight scales
    (per row and k group) and the activation scales."""
    g = torch.Generator().manual_seed(1)
    M, K, N = 48, 384, 384
    wq, ws, wdeq = quantised_weights(1, K, N, g, unit_scales=(stage == "unit-scales"), w_std=1.0)
    x8 = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    a_scale = None
    if stage == "act-scales":
        a_scale = torch.randint(120, 134, (M, K // 32), generator=g, dtype=torch.uint8)
    sizes = torch.tensor([M], dtype=torch.int32)
    y = run_mx(x8, wq, ws, sizes, device, a_scale=a_scale, out_dtype=torch.float32, block_n=block_n)
    ref = oracle.matmul_oracle(dequant_act(x8, a_scale), wdeq, None, sizes, out_dtype=torch.float32)
    err = (y - ref).abs().max().item() / ref.abs().max().item()
    assert err < 1e-5, f"{stage}: max error relative to max|ref| = {err}"


CASES = [
    # E, K, N, sizes, T
    (4, 96, 64, [13, 0, 29, 8], 50),
    (3, 512, 256, [130, 1, 64], 200),
    (8, 2880, 384, [0, 17, 128, 129, 3, 0, 64, 255], 300),
    (5, 320, 640, [60, 25, 7, 0, 51], 90),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", ["plain", "gather", "scatter_w", "swiglu", "all"])
@pytest.mark.parametrize("acts", ["bf16", "fp8", "mxfp8"])
def test_block_scaled_grouped_gemm(case, mode, acts, device):
    E, K, N, sizes, T = case
    g = torch.Generator().manual_seed(hash((E, K, N, mode)) % 1000)
    opts = dict(plain=dict(gather=False), gather=dict(gather=True),
                scatter_w=dict(gather=True, scatter=True, weights=True), swiglu=dict(gather=True, act=True),
                all=dict(gather=True, scatter=True, weights=True, act=True))[mode]
    sizes_t = torch.tensor(sizes, dtype=torch.int32)
    M = int(sizes_t.sum())
    rows_x = T if opts.get("gather") else M
    wq, ws, wdeq = quantised_weights(E, K, N, g)
    xb = torch.randn(rows_x, K, generator=g).bfloat16()
    a_scale = None
    if acts == "bf16":
        x, xref = xb, xb.float()
    else:
        x = xb.to(torch.float8_e4m3fn)
        if acts == "mxfp8":
            a_scale = torch.randint(122, 131, (rows_x, K // 32), generator=g, dtype=torch.uint8)
        xref = dequant_act(x, a_scale)
    bias = torch.randn(E, N, generator=g) * 0.1
    gather = torch.randint(0, T, (M,), generator=g, dtype=torch.int32) if opts.get("gather") else None
    scatter = torch.randperm(M, generator=g).int() if opts.get("scatter") else None
    gammas = torch.rand(M, generator=g) if opts.get("weights") else None
    betas = torch.rand(M, generator=g) if opts.get("weights") else None
    act = (1.702, 7.0) if opts.get("act") else None
    y = run_mx(x, wq, ws, sizes_t, device, a_scale=a_scale, bias=bias, gather=gather, scatter=scatter, gammas=gammas,
               betas=betas, act=act)
    ref = oracle.matmul_oracle(xref, wdeq, bias, sizes_t, gather, None, betas=betas, gammas=None if act else gammas,
                               out_dtype=torch.float32)
    if act:
        ref = oracle.swiglu_oracle(ref, *act)
        if gammas is not None:
            ref = ref * gammas[:, None]
    ref = ref.bfloat16()
    if scatter is not None:
        out = torch.zeros_like(ref)
        out[scatter.long()] = ref
        ref = out
    oracle.assert_close_oracle(ref, y, maxtol=MAXTOL_MX4, rmstol=None, what=f"block-scaled gemm {acts}")
    assert oracle.rel_l2(ref, y) < 1e-2


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", ["plain", "scatter_w", "all"])
@pytest.mark.parametrize("kernel", ["mx-f8", "mx-f4"])
def test_block_scaled_bf16_token_forms(case, mode, kernel, device):
    """bf16 tokens in each of the two forms the kernel can split them into, pinned (the automatic choice depends on
    the block size): two e4m3 terms and four e2m1 terms."""
    E, K, N, sizes, T = case
    g = torch.Generator().manual_seed(hash((E, K, N, mode)) % 1000 + 1)
    opts = dict(plain={}, scatter_w=dict(gather=True, scatter=True, weights=True),
                all=dict(gather=True, scatter=True, weights=True, act=True))[mode]
    sizes_t = torch.tensor(sizes, dtype=torch.int32)
    M = int(sizes_t.sum())
    rows_x = T if opts.get("gather") else M
    wq, ws, wdeq = quantised_weights(E, K, N, g)
    x = torch.randn(rows_x, K, generator=g).bfloat16()
    bias = torch.randn(E, N, generator=g) * 0.1
    gather = torch.randint(0, T, (M,), generator=g, dtype=torch.int32) if opts.get("gather") else None
    scatter = torch.randperm(M, generator=g).int() if opts.get("scatter") else None
    gammas = torch.rand(M, generator=g) if opts.get("weights") else None
    betas = torch.rand(M, generator=g) if opts.get("weights") else None
    act = (1.702, 7.0) if opts.get("act") else None
    y = run_mx(x, wq, ws, sizes_t, device, bias=bias, gather=gather, scatter=scatter, gammas=gammas, betas=betas, act=act,
               out_dtype=torch.float32, kernel=kernel)
    ref = oracle.matmul_oracle(x.float(), wdeq, bias, sizes_t, gather, None, betas=betas, gammas=None if act else gammas,
                               out_dtype=torch.float32)
    if act:
        ref = oracle.swiglu_oracle(ref, *act)
        if gammas is not None:
            ref = ref * gammas[:, None]
    if scatter is not None:
        out = torch.zeros_like(ref)
        out[scatter.long()] = ref
        ref = out
    # fp32 output: what is left is the split of the tokens (two e4m3 terms hold a bf16 value exactly up to underflow;
    # four e2m1 terms leave about 2^-14 of a group's maximum) and the order of the fp32 sums
    assert oracle.rel_l2(ref, y) < (5e-4 if kernel == "mx-f4" else 2e-5)


@pytest.mark.parametrize("block_m, kernel", [(16, "mx"), (32, "mx"), (64, "mx"), (16, "mx-f8"), (16, "mx-f4"), (32, "mx-f4")])
def test_block_scaled_token_block_sizes(block_m, kernel, device):
    """bf16 activations with every token-block size: experts with more rows than a block take several blocks."""
    g = torch.Generator().manual_seed(7)
    E, K, N = 6, 640, 640           # five weight blocks in groups of three: the last group of the last expert is partial
    sizes = torch.tensor([70, 1, 0, 33, 16, 5], dtype=torch.int32)
    M = int(sizes.sum())
    wq, ws, wdeq = quantised_weights(E, K, N, g)
    x = torch.randn(M, K, generator=g).bfloat16()
    y = run_mx(x, wq, ws, sizes, device, block_m=block_m, block_n=384, kernel=kernel)
    ref = oracle.matmul_oracle(x.float(), wdeq, None, sizes, out_dtype=torch.float32).bfloat16()
    oracle.assert_close_oracle(ref, y, maxtol=MAXTOL_MX4, rmstol=None, what="block-scaled gemm")
    assert oracle.rel_l2(ref, y) < 1e-2


@pytest.mark.parametrize("kernel", ["mx-f8", "mx-f4"])
def test_block_scaled_wide_dynamic_range_rows(kernel, device):
    """bf16 rows whose magnitudes span 2^40: each 32-group has its own scales, so small groups next to large ones keep
    their precision."""
    g = torch.Generator().manual_seed(9)
    E, K, N, M = 1, 512, 128, 20
    wq, ws, wdeq = quantised_weights(E, K, N, g)
    x = torch.randn(M, K, generator=g)
    x = (x * torch.exp2(torch.randint(-20, 20, (M, K // 32), generator=g).float()).repeat_interleave(32, dim=1)).bfloat16()
    sizes = torch.tensor([M], dtype=torch.int32)
    y = run_mx(x, wq, ws, sizes, device, out_dtype=torch.float32, kernel=kernel)
    ref = oracle.matmul_oracle(x.float(), wdeq, None, sizes, out_dtype=torch.float32)
    assert oracle.rel_l2(ref, y) < 1e-3


def test_block_scaled_e4m3_output(device):
    """fc1 of the fp8 mode: e4m3 rows in, SwiGLU, e4m3 rows out (saturating round to nearest)."""
    g = torch.Generator().manual_seed(21)
    E, K, N = 3, 512, 512
    sizes = torch.tensor([40, 0, 77], dtype=torch.int32)
    M = int(sizes.sum())
    wq, ws, wdeq = quantised_weights(E, K, N, g, w_std=0.05)
    x8 = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    bias = torch.randn(E, N, generator=g) * 0.1
    y = run_mx(x8, wq, ws, sizes, device, bias=bias, act=(1.702, 7.0), out_dtype=torch.float8_e4m3fn)
    assert y.dtype == torch.float8_e4m3fn
    ref32 = oracle.swiglu_oracle(oracle.matmul_oracle(x8.float(), wdeq, bias, sizes, out_dtype=torch.float32), 1.702, 7.0)
    ref8 = ref32.to(torch.float8_e4m3fn)
    # equal up to one e4m3 step where the fp32 sums differ in their last bits right at a rounding boundary
    diff = (y.float() - ref8.float()).abs()
    step = ref8.float().abs().clamp_min(2.0 ** -6) * 0.125
    assert (diff <= step).all()
    assert (diff > 0).float().mean() < 0.02


@pytest.mark.parametrize("tokens", [64, 2048])
def test_layer_with_e4m3_activations_against_oracle(tokens, device):
    """The layer in fp8 mode (e4m3 tokens in, e4m3 between the GEMMs) against the oracle fed the same quantised rows."""
    from triton_b200.moe import moe_layer_forward
    from triton_b200.testing import make_synthetic_layer
    E, k = 16, 4
    lw = make_synthetic_layer(E, 2880, 2880, device, seed=5, keep_canonical=True, block_scaled=True)
    g = torch.Generator(device=device).manual_seed(tokens)
    x8 = torch.randn(tokens, 2880, device=device, generator=g).to(torch.float8_e4m3fn)
    logits = torch.randn(tokens, E, device=device, generator=g)
    z = moe_layer_forward(x8, logits, lw, k)
    tb.matmul_check_status()
    assert z.dtype == torch.bfloat16
    rows = torch.linspace(0, tokens - 1, 6).round().long().unique()

    def expert_weights(e):
        w1 = oracle.dequant_weight_oracle(lw.w1_q[e:e + 1].cpu(), lw.w1_s[e:e + 1].cpu())[0]
        w2 = oracle.dequant_weight_oracle(lw.w2_q[e:e + 1].cpu(), lw.w2_s[e:e + 1].cpu())[0]
        return w1, lw.b1[e].cpu(), w2, lw.b2[e].cpu()

    ref = oracle.moe_layer_tokens_oracle(x8[rows.to(device)].cpu().float(), logits[rows.to(device)].cpu(), expert_weights, k,
                                         1.702, 7.0, h_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16)
    got = z[rows.to(device)].cpu()
    oracle.assert_close_oracle(ref, got, maxtol=MAXTOL_MX4, rmstol=None, what="fp8 layer")
    assert oracle.rel_l2(ref, got) < 1e-2


@pytest.mark.parametrize("K", [384, 640, 2880])
@pytest.mark.parametrize("sizes", [[3, 0, 1, 16, 0, 7], [1], [16, 16, 5, 2], [20, 1, 0, 33]])
@pytest.mark.parametrize("act", [False, True])
def test_block_scaled_few_tiles_k_step_stages(K, sizes, act, device):
    """Decode-sized calls with so few tiles that a CTA gets single weight blocks: the kernel then puts three k steps of
    one block into a stage (K = 384: exactly one stage; 640: a full and a partial one; 2880: seven and a partial one)."""
    g = torch.Generator().manual_seed(K + len(sizes) * 7 + int(act))
    E, N = len(sizes), 640
    sizes_t = torch.tensor(sizes, dtype=torch.int32)
    M = int(sizes_t.sum())
    wq, ws, wdeq = quantised_weights(E, K, N, g)
    x = torch.randn(M, K, generator=g).bfloat16()
    bias = torch.randn(E, N, generator=g) * 0.1
    gammas = torch.rand(M, generator=g)
    scatter = torch.randperm(M, generator=g).int()
    a = (1.702, 7.0) if act else None
    ref = oracle.matmul_oracle(x.float(), wdeq, bias, sizes_t, None, None, gammas=None if act else gammas, out_dtype=torch.float32)
    if act:
        ref = oracle.swiglu_oracle(ref, *a) * gammas[:, None]
    out = torch.zeros_like(ref)
    out[scatter.long()] = ref
    y = run_mx(x, wq, ws, sizes_t, device, bias=bias, scatter=scatter, gammas=gammas, act=a, out_dtype=torch.float32,
               kernel="mx-f4", block_m=16)
    assert oracle.rel_l2(out, y) < 5e-4
