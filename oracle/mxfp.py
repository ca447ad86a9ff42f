"""CPU oracle for the MXFP4 quantiser / dequantiser (TEST INFRASTRUCTURE ONLY).

Follows ``numerics_details/mxfp.py:192-343`` (``downcast_to_mxfp_torch``) and
``numerics_details/mxfp.py:346-429`` (``cvt_e2m1_to_fp32`` / ``upcast_from_mxfp_torch``)
of the reference's ``triton_kernels`` package, restricted to the format the MoE
path uses: e2m1 values packed two per byte, one e8m0 scale byte per 32 elements.
"""
import numpy as np
import torch

MX_BLOCK = 32
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
ROUND_UP, ROUND_DOWN = 0, 1


def _as_f32_last(x: torch.Tensor, axis: int):
    axis = axis % x.ndim
    return x.transpose(axis, -1).to(torch.float32).contiguous(), axis


def _e2m1_rtne_codes(q: np.ndarray) -> np.ndarray:
    """fp32 array -> 4-bit e2m1 codes (sign in bit 3), round-to-nearest-even, saturating.

    Bit-level statement of mxfp.py:287-315: the fp32 mantissa is shifted into an
    e2m1 frame (exponent bias 1, one mantissa bit), the bit below the kept
    mantissa bit is the guard, everything below it (including bits shifted out
    while denormalising) is sticky.
    """
    bits = q.view(np.uint32).astype(np.int64)
    sign = (bits >> 31) & 1
    exp = (bits >> 23) & 0xFF
    man = bits & 0x7FFFFF
    sub = exp < 127                       # |q| < 1: e2m1 subnormal range
    shift = np.clip(126 - exp, 0, 31)     # how far the implicit-1 mantissa is pushed down
    man_pre = 0x400000 | (man >> 1)       # implicit one made explicit
    lost = (man & 1) | ((man_pre & ((np.int64(1) << shift) - 1)) != 0)
    man2 = np.where(sub, man_pre >> shift, man)
    sticky = (sub & (lost != 0)) | ((man2 & 0x1FFFFF) != 0)
    e2 = np.maximum(exp, 126) - 126
    top = (man2 >> 21) & 3                # kept mantissa bit + guard bit
    keep_lsb = (top >> 1) & 1
    guard = top & 1
    inc = guard & (sticky.astype(np.int64) | keep_lsb)
    mag = np.minimum((((e2 << 2) | top) + inc) >> 1, 7)
    return ((sign << 3) | mag).astype(np.uint8)


def downcast_to_mxfp_oracle(x: torch.Tensor, axis: int, rounding_mode: int = ROUND_UP):
    """bf16/fp16/fp32 tensor -> (packed e2m1 uint8, e8m0 scale uint8), quantised along `axis`.

    Output shapes follow mxfp.py:61-64: values have ``shape[axis] // 2`` bytes along
    `axis`, scales ``shape[axis] // 32``.  Returned tensors are logically indexed
    like the input (no particular memory order is promised by the oracle).
    """
    src, axis = _as_f32_last(x, axis)
    L = src.shape[-1]
    assert L % 2 == 0
    if src.numel() == 0:
        lead = tuple(src.shape[:-1])
        return (torch.empty(lead + (L // 2,), dtype=torch.uint8).transpose(axis, -1),
                torch.empty(lead + ((L + MX_BLOCK - 1) // MX_BLOCK,), dtype=torch.uint8).transpose(axis, -1))
    pad = (-L) % MX_BLOCK
    a = src.numpy()
    lead = a.shape[:-1]
    absv = np.abs(a)
    if pad:
        a = np.concatenate([a, np.zeros(lead + (pad,), np.float32)], -1)
        absv = np.concatenate([absv, -np.ones(lead + (pad,), np.float32)], -1)
    g = absv.reshape(lead + (-1, MX_BLOCK)).max(-1)
    if rounding_mode == ROUND_UP:
        ds = (g / np.float32(6.0)).astype(np.float32)                 # mxfp.py:263
        u = (ds.view(np.uint32) + np.uint32(0x007FFFFF)) & np.uint32(0x7F800000)   # mxfp.py:270
    else:
        ds = (g / np.float32(4.0)).astype(np.float32)                 # mxfp.py:265
        u = ds.view(np.uint32) & np.uint32(0x7F800000)                # mxfp.py:272
    ds_r = u.view(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(ds_r == 0, np.float32(0), np.float32(1.0) / ds_r).astype(np.float32)
    q = (a.reshape(lead + (-1, MX_BLOCK)) * inv[..., None]).astype(np.float32)
    q = np.ascontiguousarray(q.reshape(lead + (-1,))[..., :L])
    codes = _e2m1_rtne_codes(q)
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)               # mxfp.py:317-322
    scale = (u >> 23).astype(np.uint8)                                # mxfp.py:326
    qv = torch.from_numpy(np.ascontiguousarray(packed)).transpose(axis, -1)
    sc = torch.from_numpy(np.ascontiguousarray(scale)).transpose(axis, -1)
    return qv, sc


def upcast_from_mxfp_oracle(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype, axis: int):
    """(packed e2m1 uint8, e8m0 uint8) -> `dtype`, dequantised along `axis` (mxfp.py:364-429).

    The fp32 product of the e2m1 value and 2^(byte-127) is clamped to the finite
    range of `dtype` and then cast; a scale byte of 0 is the bit pattern 0 << 23,
    i.e. +0.0 (so the whole block dequantises to zero), as in the reference; a scale
    byte of 0xFF turns its whole group into NaN.
    """
    axis = axis % q.ndim
    qn = q.transpose(axis, -1).contiguous().numpy()
    sn = scale.transpose(axis, -1).contiguous().numpy()
    lut = np.array(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), np.float32)
    vals = np.empty(qn.shape[:-1] + (qn.shape[-1] * 2,), np.float32)
    vals[..., 0::2] = lut[qn & 0xF]
    vals[..., 1::2] = lut[qn >> 4]
    L = vals.shape[-1]
    if vals.size == 0:
        return torch.from_numpy(vals).to(dtype).transpose(axis, -1).contiguous()
    s = (sn.astype(np.uint32) << 23).view(np.float32)
    pad = (-L) % MX_BLOCK
    if pad:
        vals = np.concatenate([vals, np.zeros(vals.shape[:-1] + (pad,), np.float32)], -1)
    with np.errstate(over="ignore", invalid="ignore"):
        out = vals.reshape(vals.shape[:-1] + (-1, MX_BLOCK)) * s[..., None]
    fi = torch.finfo(dtype)
    out = np.clip(out, np.float32(fi.min), np.float32(fi.max))
    # the e8m0 byte 0xFF encodes NaN: the reference's kernel overwrites the whole group
    # (mxfp_details/_upcast_from_mxfp.py:85), where its torch restatement leaves +-max and NaN only for zero codes
    out = np.where((sn == 0xFF)[..., None], np.float32(np.nan), out).reshape(vals.shape)[..., :L]
    t = torch.from_numpy(np.ascontiguousarray(out)).to(dtype)
    return t.transpose(axis, -1)
