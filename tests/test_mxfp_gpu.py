"""MXFP4 quantiser / dequantiser on the GPU, through the Python API (one C-ABI call each), bit-exact
against the fixtures made by the reference and against the CPU oracle."""
import pytest
import torch

import oracle
from triton_b200 import DequantScaleRoundingMode, downcast_to_mxfp, upcast_from_mxfp

pytestmark = pytest.mark.gpu
MODES = {0: DequantScaleRoundingMode.ROUND_UP, 1: DequantScaleRoundingMode.ROUND_DOWN}
CASES = ["mxfp_bf16_last", "mxfp_bf16_axis1", "mxfp_fp16_axis0_down", "mxfp_fp32_last", "mxfp_bf16_outliers"]


def bits(t):
    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


@pytest.mark.parametrize("name", CASES)
def test_against_reference_fixture(golden, name, device):
    g = golden(name)
    q, s = downcast_to_mxfp(g["x"].to(device), torch.uint8, g["axis"], DEQUANT_SCALE_ROUNDING_MODE=MODES[g["mode"]])
    assert q.shape == g["q"].shape and s.shape == g["scale"].shape
    assert q.stride(g["axis"]) == 1 or q.shape[g["axis"]] == 1
    assert torch.equal(q.cpu(), g["q"])
    assert torch.equal(s.cpu(), g["scale"])
    for tname, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)):
        d = upcast_from_mxfp(g["q"].to(device), g["scale"].to(device), dt, g["axis"])
        assert d.is_contiguous()
        assert torch.equal(bits(d.cpu()), bits(g["deq_" + tname]))


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
def test_rtne_known_answers(dt, device):
    # reference tests/test_mxfp.py:92-151
    above = {torch.bfloat16: 0.251953125, torch.float16: 0.250244140625, torch.float32: 0.2500000298023223877}[dt]
    x = torch.tensor([6, 0, 0.24, 0.25, 0.75, 0.99, 1.2, 1.3, -1.25, above] + [0] * 22, dtype=dt, device=device)
    x = x.view(1, -1, 1)
    q, s = downcast_to_mxfp(x, torch.uint8, axis=1)
    d = upcast_from_mxfp(q, s, dt, axis=1)
    assert d.flatten().tolist() == [6, 0, 0, 0.0, 1.0, 1.0, 1.0, 1.5, -1.0, 0.5] + [0] * 22
    x = torch.tensor([33.0, 24.0, 16.0, 8.0, 4.0, 0.0, -32.0, 0.0] + [0] * 24, device=device).bfloat16().view(1, -1, 1)
    q, s = downcast_to_mxfp(x, torch.uint8, axis=1, DEQUANT_SCALE_ROUNDING_MODE=DequantScaleRoundingMode.ROUND_DOWN)
    assert s.item() == 127 + 3
    d = upcast_from_mxfp(q, s, dt, axis=1)
    assert torch.equal(d[0, 1:].float(), x[0, 1:].float())


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
def test_extreme_values_and_exact_round_trip(dt, device):
    # reference tests/test_mxfp.py:154-205
    big = 65470 if dt == torch.float16 else 3.3895e38
    x = torch.tensor([big, big] + [0] * 30, dtype=dt, device=device)
    q, s = downcast_to_mxfp(x, torch.uint8, axis=-1)
    d = upcast_from_mxfp(q, s, dt, axis=-1)
    assert not d.isinf().any()
    assert torch.equal(bits(d.cpu()), bits(oracle.upcast_from_mxfp_oracle(q.cpu(), s.cpu(), dt, -1).contiguous()))
    vals = torch.tensor(oracle.E2M1_VALUES, dtype=dt, device=device)
    kdim = torch.cat([vals, -vals]).reshape(-1, 1)
    scales = (2.0 ** torch.arange(-8, 8, dtype=dt, device=device)).reshape(1, -1)
    w = (kdim * scales).repeat(9, 32).unsqueeze(0)
    w = w.mT.contiguous().mT
    w = torch.nn.functional.pad(w, (0, 0, 0, 16))
    q, s = downcast_to_mxfp(w, torch.uint8, axis=1)
    assert torch.equal(upcast_from_mxfp(q, s, dt, axis=1), w)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_upcast_every_scale_byte_and_code(dt, device):
    """All 256 e8m0 bytes x all 16 e2m1 codes: zero scale, denormal results, saturation at the largest scales and the
    NaN byte, bit for bit against the oracle."""
    codes = torch.arange(16, dtype=torch.uint8)
    row = (codes | (codes.flip(0) << 4)).repeat(1)            # 16 bytes = 32 codes, every code in both nibbles
    q = row.repeat(256, 1)                                    # one 32-group per scale byte
    s = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(256, 1)
    want = oracle.upcast_from_mxfp_oracle(q, s, dt, axis=1)
    got = upcast_from_mxfp(q.to(device), s.to(device), dt, axis=1).cpu()
    nan = torch.isnan(want.float())
    assert torch.equal(torch.isnan(got.float()), nan)
    assert torch.equal(bits(want.contiguous())[~nan], bits(got.contiguous())[~nan])


def test_pitched_input(device):
    # reference tests/test_mxfp.py:208-220
    torch.manual_seed(0)
    dense = torch.randn((64, 128), device=device, dtype=torch.bfloat16)
    pitched = torch.empty_strided(dense.shape, (256, 1), device=device, dtype=dense.dtype)
    pitched.copy_(dense)
    q, s = downcast_to_mxfp(pitched, torch.uint8, axis=-1)
    q2, s2 = downcast_to_mxfp(dense, torch.uint8, axis=-1)
    assert torch.equal(q, q2) and torch.equal(s, s2)


@pytest.mark.parametrize("shape, axis, mode, dt", [
    ((0, 4096, 1024), 1, 0, torch.bfloat16),
    ((3, 4096, 0), 1, 1, torch.bfloat16),
    ((3, 4096, 1024), 1, 0, torch.bfloat16),
    ((32, 254, 60), 0, 1, torch.float16),
    ((2, 16, 512), -1, 0, torch.float32),
    ((1000, 704), 1, 0, torch.bfloat16),
    ((704, 1000), 0, 0, torch.bfloat16),
])
def test_random_shapes_against_oracle(shape, axis, mode, dt, device):
    # reference tests/test_mxfp.py:223-291
    torch.manual_seed(0)
    x = torch.randn(shape, dtype=torch.float32)
    span = 6 if dt == torch.float16 else 20            # keep fp16 inputs finite: Inf / NaN inputs are not pinned
    x = (x * torch.exp2(torch.randint(-span, span, shape).float() * (torch.rand(shape) < 0.05))).to(dt)
    assert torch.isfinite(x.float()).all()
    q, s = downcast_to_mxfp(x.to(device), torch.uint8, axis, DEQUANT_SCALE_ROUNDING_MODE=MODES[mode])
    qo, so = oracle.downcast_to_mxfp_oracle(x, axis, mode)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    d = upcast_from_mxfp(q, s, dt, axis)
    do = oracle.upcast_from_mxfp_oracle(qo, so, dt, axis)
    assert torch.equal(bits(d.cpu()), bits(do.contiguous()))


def test_full_size_properties(device):
    """bf16 [8192, 8192], N(0,1) with 1 % of entries x100: checked through size-independent properties --
    a sample of rows against the oracle, idempotence of quantise(dequantise(.)), scales never clip."""
    torch.manual_seed(0)
    x = torch.randn(8192, 8192, device=device, dtype=torch.bfloat16)
    x = torch.where(torch.rand(8192, 8192, device=device) < 0.01, x * 100, x)
    q, s = downcast_to_mxfp(x, torch.uint8, axis=-1)
    d = upcast_from_mxfp(q, s, torch.bfloat16, axis=-1)
    rows = torch.arange(0, 8192, 257, device=device)
    qo, so = oracle.downcast_to_mxfp_oracle(x[rows].cpu(), -1)
    assert torch.equal(q[rows].cpu(), qo) and torch.equal(s[rows].cpu(), so)
    q2, s2 = downcast_to_mxfp(d, torch.uint8, axis=-1)
    d2 = upcast_from_mxfp(q2, s2, torch.bfloat16, axis=-1)
    assert torch.equal(d2, d)                                    # the quantised grid is a fixed point
    blk = x.float().abs().view(8192, -1, 32).amax(-1)
    dq = d.float().abs().view(8192, -1, 32).amax(-1)
    # the block maximum lands in (3, 6] after scaling and rounds to 3, 4 or 6: within [0.8, 1.2] of itself
    assert (dq <= blk * 1.2001).all() and (dq >= blk * 0.7999).all()
    err = (d.float() - x.float()).abs().view(8192, -1, 32) / blk.clamp_min(1e-30).unsqueeze(-1)
    assert err.max() <= 1.0 / 3 + 1e-6                           # half the coarsest e2m1 step (4 -> 6), block max > 3
