"""Masked / scaled sum over one axis of a 3-D tensor: the combine of the k expert outputs of a token
(triton_kernels/reduce.py:664-853, 1143-1165).  Forward only; mx / flexpoint / post-process hooks of the
reference are not part of the MoE path and raise NotImplementedError."""
from typing import Optional

import torch

from . import _lib


def _strides3(t, shape, dim):
    """element strides of `t` broadcast to `shape`, ordered (reduced, s0, s1); 0 where broadcast."""
    if t.ndim != 3:
        t = t.reshape((1,) * (3 - t.ndim) + tuple(t.shape))
    st = [0 if t.shape[i] == 1 and shape[i] != 1 else t.stride(i) for i in range(3)]
    for i in range(3):
        assert t.shape[i] in (1, shape[i]), f"cannot broadcast {tuple(t.shape)} to {tuple(shape)}"
    nonred = [d for d in range(3) if d != dim]
    return st[dim], st[nonred[0]], st[nonred[1]]


def reduce(x: torch.Tensor, dim: int, mask: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None,
           x_mxscale=None, x_flex=None, x_global_scale=None, y: Optional[torch.Tensor] = None,
           y_dtype: Optional[torch.dtype] = None, y_flex=None, y_flex_saturate_inf: bool = False, y_has_mx=None,
           y_mx_scale_dtype=None, y_microblock_size: int = 32, y_value_pack_factor: int = 1, postprocess_fn1=None,
           postprocess_fn2=None, unpadded_batch_size=None):
    """-> (y, None) with y[s0, s1] = sum over `dim` of where(mask != 0, x * scale, 0), fp32 accumulation,
    cast to `y_dtype` (default x.dtype).  `mask` / `scale` broadcast against x."""
    if x.ndim != 3:
        raise NotImplementedError("reduce only supports 3D inputs in this implementation")
    if dim < 0:
        dim += x.ndim
    if dim not in (0, 1, 2):
        raise ValueError("dim must be in {0,1,2}")
    for name, v in (("x_mxscale", x_mxscale), ("x_global_scale", x_global_scale), ("postprocess_fn1", postprocess_fn1),
                    ("postprocess_fn2", postprocess_fn2), ("unpadded_batch_size", unpadded_batch_size)):
        if v is not None:
            raise NotImplementedError(f"reduce: {name} is not supported")
    if y_has_mx or (x_flex is not None and x_flex.scale is not None) or \
            (y_flex is not None and y_flex.expected_scale is not None):
        raise NotImplementedError("reduce: mx / flexpoint outputs are not supported")
    lib = _lib.load()
    nonred = [d for d in range(3) if d != dim]
    S0, S1, R = x.shape[nonred[0]], x.shape[nonred[1]], x.shape[dim]
    y_dtype = y_dtype or x.dtype
    if y is None:
        y = torch.empty((S0, S1), device=x.device, dtype=y_dtype)
    assert tuple(y.shape) == (S0, S1)
    if S0 == 0 or S1 == 0:
        return y, None
    sm = (0, 0, 0)
    mbytes = 0
    if mask is not None:
        if mask.dtype == torch.bool:
            mask = mask.view(torch.uint8)
        elif mask.dtype.is_floating_point:
            mask = (mask != 0).view(torch.uint8)
        mbytes = mask.element_size()
        sm = _strides3(mask, x.shape, dim)
    ss = (0, 0, 0)
    if scale is not None:
        if scale.dtype != torch.float32:
            scale = scale.float()
        ss = _strides3(scale, x.shape, dim)
    _lib.check(lib.moe_reduce(_lib.ptr(x), _lib.dtype_code(x.dtype), R, S0, S1, x.stride(dim), x.stride(nonred[0]),
                              x.stride(nonred[1]), _lib.ptr(mask), mbytes, *sm, _lib.ptr(scale), *ss, _lib.ptr(y),
                              _lib.dtype_code(y.dtype), y.stride(0), y.stride(1), _lib.stream()), "moe_reduce")
    return y, None
