"""Standalone SwiGLU on interleaved gate/linear columns (triton_kernels/swiglu.py:10-100).  The fused
form is selected in `matmul` through `FusedActivation(FnSpecs("swiglu", swiglu_fn, ...), (alpha, limit))`."""
from dataclasses import dataclass

import torch

from . import _lib
from .numerics import InFlexData, OutFlexData


@dataclass(frozen=True)
class FlexCtx:
    out_data: OutFlexData = OutFlexData()
    inp_data: InFlexData = InFlexData()
    saturate_inf: bool = False


@dataclass(frozen=True)
class PrecisionConfig:
    limit: float | None
    flex_ctx: FlexCtx = FlexCtx()


def swiglu_fn(input, alpha, limit):
    """Marker for the fused activation: `matmul` recognises FnSpecs named "swiglu" and runs the SwiGLU
    epilogue of the CUDA kernel.  It is never called on the host."""
    raise RuntimeError("swiglu_fn is a fusion marker; call swiglu() for the standalone operator")


def swiglu(a, alpha, precision_config, routing_data=None, n_rows=None):
    """a [..., 2N] -> [..., N]: out = s * (linear + 1), s = gate * sigmoid(alpha * gate), gate = even columns
    clamped to <= limit, linear = odd columns clamped to [-limit, limit].  `n_rows` (device int32 scalar)
    optionally bounds the rows that are computed."""
    lib = _lib.load()
    fc = precision_config.flex_ctx
    if fc.inp_data.scale is not None or fc.out_data.expected_scale is not None:
        raise NotImplementedError("flexpoint scales are not supported by swiglu")
    N2 = a.shape[-1]
    assert N2 % 2 == 0 and a.stride(-1) == 1
    M = a.numel() // N2 if N2 else 0
    a2 = a.reshape(M, N2)
    out = torch.empty((M, N2 // 2), dtype=a.dtype, device=a.device)
    limit = precision_config.limit
    _lib.check(lib.moe_swiglu(_lib.ptr(a2), a2.stride(0), _lib.ptr(out), out.stride(0), _lib.dtype_code(a.dtype), M,
                              N2 // 2, float(alpha), float(limit if limit is not None else 0.0), int(limit is not None),
                              _lib.ptr(n_rows), _lib.stream()), "moe_swiglu")
    return out.view(a.shape[:-1] + (N2 // 2,))
