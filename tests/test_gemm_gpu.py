"""Ragged grouped GEMM on the GPU against the CPU oracle: the SIMT kernel (canonical / dense weights) and
the tcgen05 kernel (B200 tiled weights), with gather, scatter, bias, betas / gammas, SwiGLU."""
import pytest
import torch

import oracle
import triton_b200 as tb
from triton_b200.tensor import FP4, convert_layout, wrap_torch_tensor
from triton_b200.tensor_details.layout import (B200MXScaleLayout, B200MXValueLayout, BlackwellMXScaleLayout,
                                               BlackwellMXValueLayout)

pytestmark = pytest.mark.gpu

# tolerance of the reference's tests for MXFP4 weights: tests/test_matmul.py:649-650 (max 3e-2, rms unchecked);
# in addition the relative L2 error must stay below 1e-2
MAXTOL_MX4 = 3e-2


def make_problem(E, K, N, sizes, T, seed, device, act=False, gather=True, scatter=False, bias=True, weights=False,
                 w_std=0.02):
    g = torch.Generator().manual_seed(seed)
    sizes = torch.tensor(sizes, dtype=torch.int32)
    M = int(sizes.sum())
    x = torch.randn(T if gather else M, K, generator=g).bfloat16()
    w = (torch.randn(E, K, N, generator=g) * w_std).bfloat16()
    wq, ws = oracle.downcast_to_mxfp_oracle(w, 1)
    wq, ws = wq.contiguous().transpose(1, 2).contiguous().transpose(1, 2), ws.contiguous().transpose(1, 2).contiguous().transpose(1, 2)
    p = dict(E=E, K=K, N=N, M=M, sizes=sizes, x=x, wq=wq, ws=ws)
    p["bias"] = torch.randn(E, N, generator=g) * 0.1 if bias else None
    p["gather"] = torch.randint(0, T, (M,), generator=g, dtype=torch.int32) if gather else None
    p["scatter"] = torch.randperm(M, generator=g).int() if scatter else None
    p["gammas"] = torch.rand(M, generator=g) if weights else None
    p["betas"] = torch.rand(M, generator=g) if weights else None
    p["act"] = (1.702, 7.0) if act else None
    p["wdeq"] = oracle.dequant_weight_oracle(wq, ws)
    return p


def reference(p, fp32_act=True):
    y = oracle.matmul_oracle(p["x"], p["wdeq"], p["bias"], p["sizes"], p["gather"], None, betas=p["betas"],
                             gammas=None if p["act"] else p["gammas"], out_dtype=torch.float32)
    if p["act"]:
        y = oracle.swiglu_oracle(y, *p["act"])
        if p["gammas"] is not None:
            y = y * p["gammas"][:, None]
    y = y.bfloat16()
    if p["scatter"] is not None:
        out = torch.zeros_like(y)
        out[p["scatter"].long()] = y
        y = out
    return y


def run(p, device, layout, kernel="auto", block_m=None, block_n=None):
    dev = lambda t: None if t is None else t.to(device)
    wq = wrap_torch_tensor(dev(p["wq"]), dtype=FP4)
    ws = wrap_torch_tensor(dev(p["ws"]))
    assert wq.shape == [p["E"], p["K"], p["N"]]
    if layout == "b200":
        wq, ws = convert_layout(wq, B200MXValueLayout()), convert_layout(ws, B200MXScaleLayout())
    elif layout == "blackwell":
        wq, ws = convert_layout(wq, BlackwellMXValueLayout()), convert_layout(ws, BlackwellMXScaleLayout())
    md = tb.make_ragged_tensor_metadata(dev(p["sizes"]), p["M"])
    pc = tb.PrecisionConfig(b_mx_scale=ws, b_microblock_size=32)
    fa = None
    if p["act"]:
        fa = tb.FusedActivation(tb.FnSpecs("swiglu", tb.swiglu_fn, ("alpha", "limit"), reduction_n=2), p["act"])
    cons = {"kernel": kernel}
    if block_m:
        cons["block_m"] = block_m
    if block_n:
        cons["block_n"] = block_n
    with tb.scoped_opt_flags_constraints(cons):
        y = tb.matmul(dev(p["x"]), wq, dev(p["bias"]), md, None, dev(p["gather"]), dev(p["scatter"]), pc,
                      betas=dev(p["betas"]), gammas=dev(p["gammas"]), fused_activation=fa)
    tb.matmul_check_status()
    return y


def check(p, y, scatter_valid=None):
    ref = reference(p)
    got = y.cpu()
    if p["scatter"] is None:
        n = p["M"]
        ref, got = ref[:n], got[:n]
    oracle.assert_close_oracle(ref, got, maxtol=MAXTOL_MX4, rmstol=None, what="gemm")
    assert oracle.rel_l2(ref, got) < 1e-2


SMALL = [
    # E, K, N, sizes, T
    (4, 96, 64, [13, 0, 29, 8], 50),
    (1, 64, 32, [5], 9),
    (3, 512, 256, [130, 1, 64], 200),
    (8, 2880, 384, [0, 17, 128, 129, 3, 0, 64, 255], 300),
    (5, 320, 128, [600, 256, 257, 0, 511], 700),
]


@pytest.mark.parametrize("case", SMALL)
@pytest.mark.parametrize("mode", ["plain", "gather", "scatter_w", "swiglu", "all"])
@pytest.mark.parametrize("path", ["simt-canonical", "simt-blackwell", "tcgen05", "tcgen05-256", "tcgen05-256x256", "tcgen05-pair", "stream"])
def test_grouped_gemm(case, mode, path, device):
    E, K, N, sizes, T = case
    opts = dict(plain=dict(gather=False), gather=dict(gather=True),
                scatter_w=dict(gather=True, scatter=True, weights=True), swiglu=dict(gather=True, act=True),
                all=dict(gather=True, scatter=True, weights=True, act=True))[mode]
    p = make_problem(E, K, N, sizes, T, seed=hash((E, K, N, mode)) % 1000, device=device, **opts)
    layout, kernel, block_m, block_n = {
        "simt-canonical": ("canonical", "simt", None, None), "simt-blackwell": ("blackwell", "simt", None, None),
        "tcgen05": ("b200", "tcgen05", 128, 128), "tcgen05-256": ("b200", "tcgen05", 256, 128),
        "tcgen05-256x256": ("b200", "tcgen05", 256, 256), "tcgen05-pair": ("b200", "tcgen05-pair", 0, 0), "stream": ("b200", "stream", 0, 0)}[path]
    y = run(p, device, layout, kernel, block_m, block_n)
    check(p, y)


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05-pair"])
@pytest.mark.parametrize("mode", ["gather", "all"])
def test_grouped_gemm_pregathered_rows(kernel, mode, device):
    """2048+ gathered rows with large experts: the rows are first copied into the scratch buffer the host passes and
    the kernel streams them by TMA tile copies."""
    opts = dict(gather=dict(gather=True), all=dict(gather=True, scatter=True, weights=True, act=True))[mode]
    p = make_problem(4, 320, 256, [900, 700, 385, 127], 800, seed=11, device=device, **opts)
    y = run(p, device, "b200", kernel, 0, 0)
    check(p, y)


@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
@pytest.mark.parametrize("sizes, T", [([13, 0, 29, 8], 50), ([600, 256, 257, 511], 700)])
def test_fused_comm_block_rows(kernel, sizes, T, device):
    """Output rows spread over three buffers (here all on one device): row r of the scattered output lands in row
    r % rows_per_shard of buffer r // rows_per_shard."""
    p = make_problem(4, 320, 128, sizes, T, seed=5, device=device, gather=True, scatter=True, weights=True)
    M = p["M"]
    shards = 3
    rows_per_shard = (M + shards - 1) // shards
    bufs = [torch.zeros(rows_per_shard, 128, dtype=torch.bfloat16, device=device) for _ in range(shards)]
    dev = lambda t: None if t is None else t.to(device)
    layout = "canonical" if kernel == "simt" else "b200"
    wq = wrap_torch_tensor(dev(p["wq"]), dtype=FP4)
    ws = wrap_torch_tensor(dev(p["ws"]))
    if layout == "b200":
        wq, ws = convert_layout(wq, B200MXValueLayout()), convert_layout(ws, B200MXScaleLayout())
    md = tb.make_ragged_tensor_metadata(dev(p["sizes"]), M)
    pc = tb.PrecisionConfig(b_mx_scale=ws, b_microblock_size=32)
    fc = tb.FusedComm([b.data_ptr() for b in bufs], rows_per_shard, bufs[0])
    with tb.scoped_opt_flags_constraints({"kernel": kernel}):
        y0 = tb.matmul(dev(p["x"]), wq, dev(p["bias"]), md, None, dev(p["gather"]), dev(p["scatter"]), pc,
                       betas=dev(p["betas"]), gammas=dev(p["gammas"]), fused_comm=fc)
    tb.matmul_check_status()
    assert y0.data_ptr() == bufs[0].data_ptr()
    y = torch.cat(bufs)[:M]
    check(p, y)


def test_against_reference_fixture(golden, device):
    g = golden("gemm_small")
    wq = wrap_torch_tensor(g["wq"].to(device).transpose(1, 2).contiguous().transpose(1, 2), dtype=FP4)
    ws = wrap_torch_tensor(g["ws"].to(device).transpose(1, 2).contiguous().transpose(1, 2))
    md = tb.make_ragged_tensor_metadata(g["slice_sizes"].to(device), 50)
    for layout in ("canonical", "b200"):
        wq2, ws2 = wq, ws
        if layout == "b200":
            wq2, ws2 = convert_layout(wq, B200MXValueLayout()), convert_layout(ws, B200MXScaleLayout())
        pc = tb.PrecisionConfig(b_mx_scale=ws2, b_microblock_size=32)
        y = tb.matmul(g["x"].to(device), wq2, g["bias"].to(device), md, None, g["gather"].to(device),
                      g["scatter"].to(device), pc, gammas=g["gammas"].to(device))
        tb.matmul_check_status()
        oracle.assert_close_oracle(g["y"], y.cpu(), maxtol=MAXTOL_MX4, rmstol=None, what=layout)


def test_dense_plain_product_library_gemm(device):
    """x @ W + b without routing (the router's logits) goes to the library GEMM; same answer as the SIMT kernel."""
    torch.manual_seed(1)
    x = torch.randn(300, 2880, device=device).bfloat16()
    w = (torch.randn(2880, 128, device=device) * 0.02).bfloat16()
    b = torch.randn(128, device=device)
    y = tb.matmul(x, w, b)
    with tb.scoped_opt_flags_constraints({"kernel": "simt"}):
        y_simt = tb.matmul(x, w, b)
    ref = (x.float().cpu() @ w.float().cpu() + b.cpu()).bfloat16()
    oracle.assert_close_oracle(ref, y.cpu())
    oracle.assert_close_oracle(ref, y_simt.cpu())


def test_dense_weights_simt(device):
    torch.manual_seed(0)
    x = torch.randn(70, 100, device=device).bfloat16()
    w = (torch.randn(100, 48, device=device) * 0.1).bfloat16()
    b = torch.randn(48, device=device)
    y = tb.matmul(x, w, b)
    ref = (x.float().cpu() @ w.float().cpu() + b.cpu()).bfloat16()
    oracle.assert_close_oracle(ref, y.cpu())


def test_weight_layout_round_trip(device):
    torch.manual_seed(0)
    E, K, N = 3, 2880, 200
    q = torch.randint(0, 256, (E, K, N // 2), dtype=torch.uint8, device=device)      # canonical, packed along N
    s = torch.randint(0, 255, (E, K // 32, N), dtype=torch.uint8, device=device)
    tq, ts = wrap_torch_tensor(q, dtype=FP4), wrap_torch_tensor(s)
    assert tq.shape == [E, K, N]
    bq, bs = convert_layout(tq, B200MXValueLayout()), convert_layout(ts, B200MXScaleLayout())
    lib = tb._lib.load()
    assert bq.storage.data.numel() == lib.moe_weight_b200_value_bytes(E, K, N)
    assert bs.storage.data.numel() == lib.moe_weight_b200_scale_bytes(E, K, N)
    from triton_b200.tensor_details.layout import StridedLayout
    assert torch.equal(convert_layout(bq, StridedLayout()).storage.data, q)
    assert torch.equal(convert_layout(bs, StridedLayout()).storage.data, s)
    # through the reference's Blackwell layouts and back
    vq = convert_layout(tq, BlackwellMXValueLayout())
    assert torch.equal(convert_layout(convert_layout(vq, B200MXValueLayout()), StridedLayout()).storage.data, q)
    g_s = oracle.swizzle_mx_scale_bw_oracle(s.cpu())
    assert torch.equal(convert_layout(ts, BlackwellMXScaleLayout()).storage.data.cpu(), g_s)


@pytest.fixture(scope="module")
def layer_20b():
    """gpt-oss-20b-shaped expert weights (32 experts, d_model 2880, fused gate+up 5760) and their CPU dequantisation."""
    from triton_b200.testing import make_synthetic_layer
    lw = make_synthetic_layer(32, 2880, 2880, "cuda", seed=0, keep_canonical=True)
    w1 = oracle.dequant_weight_oracle(lw.w1_q.cpu(), lw.w1_s.cpu())
    w2 = oracle.dequant_weight_oracle(lw.w2_q.cpu(), lw.w2_s.cpu())
    return lw, w1, w2


@pytest.mark.parametrize("tokens", [1, 16, 64, 512])
def test_gpt_oss_20b_layer_against_oracle(tokens, layer_20b, device):
    """One gpt-oss-20b-shaped MoE layer (top-4, SwiGLU alpha 1.702 limit 7) against the oracle, at the token
    counts the oracle finishes in seconds."""
    from triton_b200.moe import moe_layer_forward
    lw, w1, w2 = layer_20b
    torch.manual_seed(tokens)
    x = torch.randn(tokens, 2880, device=device).bfloat16()
    logits = torch.randn(tokens, 32, device=device)
    z = moe_layer_forward(x, logits, lw, 4)
    tb.matmul_check_status()
    ref = oracle.moe_layer_oracle(x.cpu(), logits.cpu(), w1, lw.b1.cpu(), w2, lw.b2.cpu(), 4, 1.702, 7.0,
                                  fuse_activation_fp32=True)
    oracle.assert_close_oracle(ref, z.cpu(), maxtol=MAXTOL_MX4, rmstol=None, what=f"layer T={tokens}")
    assert oracle.rel_l2(ref, z.cpu()) < 1e-2


@pytest.mark.parametrize("tokens", [4096, 16384])
def test_gpt_oss_20b_layer_full_size_properties(tokens, layer_20b, device):
    """Full-size token counts, checked through properties that need no CPU GEMM: (1) the tensor-core kernel and
    the SIMT kernel (canonical weights) agree; (2) a token's output does not depend on which other tokens are in
    the batch (rows of a sub-batch reproduce bit-for-bit... up to accumulation order: within tolerance)."""
    from triton_b200.moe import moe_layer_forward, MoeLayerWeights
    lw, _, _ = layer_20b
    torch.manual_seed(tokens)
    x = torch.randn(tokens, 2880, device=device).bfloat16()
    logits = torch.randn(tokens, 32, device=device)
    z = moe_layer_forward(x, logits, lw, 4)
    tb.matmul_check_status()
    sub = torch.arange(0, tokens, 37, device=device)[:256]
    lw_c = MoeLayerWeights(wrap_torch_tensor(lw.w1_q, dtype=FP4), wrap_torch_tensor(lw.w1_s), lw.b1,
                           wrap_torch_tensor(lw.w2_q, dtype=FP4), wrap_torch_tensor(lw.w2_s), lw.b2)
    with tb.scoped_opt_flags_constraints({"kernel": "simt"}):
        z_sub = moe_layer_forward(x[sub].contiguous(), logits[sub].contiguous(), lw_c, 4)
    oracle.assert_close_oracle(z_sub.cpu(), z[sub].cpu(), maxtol=MAXTOL_MX4, rmstol=None, what="tcgen05 vs simt")
    assert oracle.rel_l2(z_sub.cpu(), z[sub].cpu()) < 1e-2
    assert torch.isfinite(z.float()).all()


@pytest.mark.parametrize("tokens", [4, 64])
def test_graphed_layer_equals_eager_layer(tokens, layer_20b, device):
    """The layer replayed from a CUDA graph returns exactly what the eager layer returns, for new inputs too."""
    from triton_b200.moe import GraphedMoeLayer, moe_layer_forward
    lw, _, _ = layer_20b
    graphed = GraphedMoeLayer(lw, 4, tokens, 2880, 32, device)
    for seed in (1, 2):
        g = torch.Generator(device=device).manual_seed(seed)
        x = torch.randn(tokens, 2880, device=device, generator=g).bfloat16()
        logits = torch.randn(tokens, 32, device=device, generator=g)
        want = moe_layer_forward(x, logits, lw, 4)
        got = graphed(x, logits).clone()
        tb.matmul_check_status()
        assert torch.equal(want, got)


def test_host_streaming_layer(layer_20b, device):
    """Steps fed from and returned to pinned host memory through the three-stream pipeline equal the eager layer."""
    from triton_b200.moe import HostStreamingLayer, moe_layer_forward
    lw, _, _ = layer_20b
    T = 300
    pipe = HostStreamingLayer(lambda x, l: moe_layer_forward(x, l, lw, 4), T, 2880, 32, device)
    xs, ls, zs, want = [], [], [], []
    for seed in range(5):
        g = torch.Generator().manual_seed(seed)
        xs.append(torch.randn(T, 2880, generator=g).bfloat16().pin_memory())
        ls.append(torch.randn(T, 32, generator=g).pin_memory())
        zs.append(torch.empty(T, 2880, dtype=torch.bfloat16).pin_memory())
        want.append(moe_layer_forward(xs[-1].to(device), ls[-1].to(device), lw, 4).cpu())
    for i in range(5):
        pipe.submit(xs[i], ls[i], zs[i])
    pipe.drain()
    torch.cuda.synchronize()
    tb.matmul_check_status()
    for i in range(5):
        assert torch.equal(zs[i], want[i]), i


def _sampled_layer_check(lw, n_expts, tokens, device, seed, skew, n_sample=8):
    """Run the layer on `tokens` tokens and compare `n_sample` of its output rows with the CPU oracle, which needs only
    the experts those rows are routed to."""
    from triton_b200.moe import moe_layer_forward
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(tokens, 2880, device=device, generator=g).bfloat16()
    logits = torch.randn(tokens, n_expts, device=device, generator=g)
    if skew:
        logits = logits + torch.randn(n_expts, device=device, generator=g)
    z = moe_layer_forward(x, logits, lw, 4)
    tb.matmul_check_status()
    rows = torch.linspace(0, tokens - 1, n_sample).round().long().unique()

    def expert_weights(e):
        w1 = oracle.dequant_weight_oracle(lw.w1_q[e:e + 1].cpu(), lw.w1_s[e:e + 1].cpu())[0]
        w2 = oracle.dequant_weight_oracle(lw.w2_q[e:e + 1].cpu(), lw.w2_s[e:e + 1].cpu())[0]
        return w1, lw.b1[e].cpu(), w2, lw.b2[e].cpu()

    ref = oracle.moe_layer_tokens_oracle(x[rows.to(device)].cpu(), logits[rows.to(device)].cpu(), expert_weights, 4, 1.702, 7.0)
    got = z[rows.to(device)].cpu()
    oracle.assert_close_oracle(ref, got, maxtol=MAXTOL_MX4, rmstol=None, what=f"layer E={n_expts} T={tokens}, sampled rows")
    assert oracle.rel_l2(ref, got) < 1e-2
    assert torch.isfinite(z.float()).all()


def test_gpt_oss_120b_layer_benchmark_configuration_against_oracle(device):
    """The benchmarked configuration itself -- 128 experts, 16384 tokens, skewed router: 256 x 256 tiles, TMA activation
    loads, row-gather scratch -- against the CPU oracle on sampled tokens."""
    from triton_b200.testing import make_synthetic_layer
    lw = make_synthetic_layer(128, 2880, 2880, device, seed=1000, keep_canonical=True)
    _sampled_layer_check(lw, 128, 16384, device, seed=0, skew=True)


@pytest.mark.parametrize("tokens", [1, 16, 64, 300, 1200])
def test_gpt_oss_120b_layer_decode_path_against_oracle(tokens, device):
    """Steps of the 128-expert layer with up to 48 rows per expert on average take the block-scaled kernel (its own copy of
    the weights): 1 to 64 tokens in 16-row token blocks (four e2m1 terms), 300 and 1200 tokens (9 and 38 rows per expert) in
    32-row blocks (two e4m3 terms)."""
    from triton_b200.testing import make_synthetic_layer
    lw = make_synthetic_layer(128, 2880, 2880, device, seed=1000, keep_canonical=True, block_scaled=True)
    assert lw.use_block_scaled(tokens * 4)
    _sampled_layer_check(lw, 128, tokens, device, seed=tokens, skew=True, n_sample=min(tokens, 6))


def test_weight_file_and_block_checkpoint_reader(tmp_path, device):
    """A layer saved in its tiled layouts and read back computes the same output bit for bit, and the checkpoint form
    (blocks [E, N, K/32, 16] + scales [E, N, K/32]) converts to the very same tiles."""
    from triton_b200.moe import moe_layer_forward
    from triton_b200.testing import make_synthetic_layer
    from triton_b200.weights_io import from_block_checkpoint, load_layer_weights, save_layer_weights
    E, d, ff, k, T = 8, 512, 256, 2, 100
    lw = make_synthetic_layer(E, d, ff, device, seed=3, keep_canonical=True, block_scaled=True)
    path = tmp_path / "layer.moeb200w"
    save_layer_weights(path, lw)
    back = load_layer_weights(path, device)
    torch.manual_seed(1)
    x = torch.randn(T, d, device=device).bfloat16()
    logits = torch.randn(T, E, device=device)
    z0, z1 = moe_layer_forward(x, logits, lw, k), moe_layer_forward(x, logits, back, k)
    tb.matmul_check_status()
    assert torch.equal(z0, z1)
    # checkpoint form: canonical K-packed bytes regrouped as 16-byte blocks
    blocks1 = lw.w1_q.transpose(1, 2).contiguous().reshape(E, 2 * ff, d // 32, 16)
    blocks2 = lw.w2_q.transpose(1, 2).contiguous().reshape(E, d, ff // 32, 16)
    ck = from_block_checkpoint(blocks1, lw.w1_s.transpose(1, 2).contiguous(), lw.b1, blocks2,
                               lw.w2_s.transpose(1, 2).contiguous(), lw.b2, block_scaled=True)
    for name in ("w1", "w1_scale", "w2", "w2_scale", "w1_bs", "w1_bs_scale", "w2_bs", "w2_bs_scale"):
        assert torch.equal(getattr(ck, name).storage.data, getattr(lw, name).storage.data), name
