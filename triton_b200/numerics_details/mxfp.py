"""MXFP4 quantise / dequantise (triton_kernels/numerics_details/mxfp.py:25-176): e2m1 values packed two
per byte along `axis`, one e8m0 scale byte per 32 elements.  MXFP8 / NVFP4 variants of the reference
are outside the MoE path and raise NotImplementedError."""
from enum import Enum

import torch

from .. import _lib
from ..tensor import FP4, Tensor

MXFP_BLOCK_SIZE = 32
NVFP_BLOCK_SIZE = 16


class DequantScaleRoundingMode(Enum):
    ROUND_UP = 0      # scale = 2^ceil(log2(max / 6)): never clips the block maximum
    ROUND_DOWN = 1    # scale = 2^floor(log2(max / 4)): the OCP rule, may clip


def _collapse3(t, axis):
    """View `t` (axis moved last) as [batch, outer, quant] with element strides, copying only when the
    leading dimensions cannot be merged into two."""
    tt = t.transpose(axis, -1)
    lead = [(s, st) for s, st in zip(tt.shape[:-1], tt.stride()[:-1]) if s != 1]
    merged = []
    for s, st in lead:                       # merge adjacent dims that are contiguous with each other
        if merged and merged[-1][1] == st * s:
            merged[-1] = (merged[-1][0] * s, st)
        else:
            merged.append((s, st))
    if len(merged) > 2:
        tt = tt.contiguous()
        outer = tt.numel() // max(tt.shape[-1], 1)
        return tt, 1, outer, 0, tt.shape[-1], 1
    while len(merged) < 2:
        merged.insert(0, (1, 0))
    (b, sb), (o, so) = merged
    return tt, b, o, sb, so, tt.stride(-1)


def downcast_to_mxfp(x, out_dtype, axis: int, scale_dtype: torch.dtype = torch.uint8,
                     microblock_size: int = MXFP_BLOCK_SIZE,
                     DEQUANT_SCALE_ROUNDING_MODE: DequantScaleRoundingMode = DequantScaleRoundingMode.ROUND_UP):
    """-> (values uint8, scales uint8).  values.shape = x.shape with shape[axis] halved, scales.shape with
    shape[axis] // 32; both are contiguous along `axis` (StridedLayout(major_dim=axis), mxfp.py:61-64)."""
    if isinstance(x, Tensor):
        x = x.storage.data
    if out_dtype not in (torch.uint8, FP4):
        raise NotImplementedError("downcast_to_mxfp: only MXFP4 (torch.uint8) output is supported")
    if scale_dtype != torch.uint8 or microblock_size != MXFP_BLOCK_SIZE:
        raise NotImplementedError("downcast_to_mxfp: only e8m0 scales per 32 elements are supported")
    assert -x.ndim <= axis < x.ndim, f"Invalid axis {axis=}"
    axis %= x.ndim
    L = x.shape[axis]
    assert L % microblock_size == 0, f"axis dim must be divisible by {microblock_size}. Got {L}"
    lib = _lib.load()
    # outputs: quantised axis innermost in memory, the other axes as in x.transpose(axis, -1)
    lead = x.transpose(axis, -1).shape[:-1]
    q = torch.empty((*lead, L // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty((*lead, L // 32), dtype=torch.uint8, device=x.device)
    if x.numel() > 0:
        xt, b, o, sb, so, sq = _collapse3(x, axis)
        _lib.check(lib.moe_downcast_mxfp4(_lib.ptr(xt), _lib.dtype_code(x.dtype), b, o, L, sb, so, sq, _lib.ptr(q),
                                          _lib.ptr(s), DEQUANT_SCALE_ROUNDING_MODE.value, _lib.stream()),
                   "moe_downcast_mxfp4")
    return q.transpose(axis, -1), s.transpose(axis, -1)


def upcast_from_mxfp(tensor: torch.Tensor, scale: torch.Tensor, target_dtype: torch.dtype, axis: int,
                     tensor_scale=None):
    """Packed e2m1 + e8m0 -> fp16 / bf16 / fp32, dequantised along `axis`; result is contiguous."""
    if tensor_scale is not None:
        raise NotImplementedError("upcast_from_mxfp: tensor_scale is not supported")
    if tensor.dtype != torch.uint8 or scale.dtype != torch.uint8:
        raise NotImplementedError("upcast_from_mxfp: only MXFP4 values with e8m0 scales are supported")
    assert target_dtype in (torch.float16, torch.bfloat16, torch.float32), f"Invalid output dtype {target_dtype=}"
    ndim = tensor.ndim
    assert -ndim <= axis < ndim and tensor.ndim == scale.ndim
    axis %= ndim
    lib = _lib.load()
    q = tensor.transpose(axis, -1).contiguous()
    s = scale.transpose(axis, -1).contiguous()
    L = q.shape[-1] * 2
    assert s.shape[-1] * 32 == L, "scale shape does not match the packed values"
    out_shape = list(tensor.shape)
    out_shape[axis] = L
    out = torch.empty(out_shape, dtype=target_dtype, device=tensor.device)
    if out.numel() > 0:
        ot, b, o, sb, so, sq = _collapse3(out, axis)
        _lib.check(lib.moe_upcast_mxfp4(_lib.ptr(q), _lib.ptr(s), _lib.ptr(ot), _lib.dtype_code(target_dtype), b, o, L,
                                        sb, so, sq, _lib.stream()), "moe_upcast_mxfp4")
        if ot.data_ptr() != out.data_ptr():      # more than two non-mergeable leading axes: written to a copy
            out.transpose(axis, -1).copy_(ot)
    return out
