"""Layout catalogue and the per-device defaults (triton_kernels/tensor_details/layout.py:27-54).

On B200 the default MXFP4 weight layouts are the tile-contiguous ones the tcgen05 kernel streams; the
reference's Blackwell layouts are kept for interchange (`convert_layout` goes through the canonical
form, so any pair of layouts converts both ways)."""
from .layout_details.base import Layout
from .layout_details.strided import StridedLayout
from .layout_details.blackwell_scale import BlackwellActMXScaleLayout, BlackwellMXScaleLayout
from .layout_details.blackwell_value_shuffled import BlackwellMX4ValueShuffledLayout
from .layout_details.blackwell_value import BlackwellMXValueLayout
from .layout_details.b200_tiled import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout, B200MXScaleLayout,
                                        B200MXValueLayout)

__all__ = ["Layout", "StridedLayout", "BlackwellMXScaleLayout", "BlackwellActMXScaleLayout", "BlackwellMXValueLayout",
           "BlackwellMX4ValueShuffledLayout", "B200MXValueLayout",
           "B200MXScaleLayout", "B200BlockScaledValueLayout", "B200BlockScaledScaleLayout", "make_default_matmul_mxfp4_w_layout", "make_default_matmul_mxfp4_w_scale_layout"]


def make_default_matmul_mxfp4_w_layout(mx_axis: int = -2, allow_blackwell_value_shuffle: bool = False,
                                       block_k: int = 128, block_n: int = 256):
    """Layout the weights of an MXFP4 `matmul` should be converted to on this device
    (triton_kernels/tensor_details/layout.py:27-46).  The tensor-core kernels here stream tiles of 128 n x 128 k that are
    contiguous whatever tile the caller had in mind, so `allow_blackwell_value_shuffle`, `block_k` and `block_n` -- the
    reference's choice between its plain and its pre-tiled Blackwell layout -- select nothing; weights that were
    prepared in either of those layouts convert with `convert_layout`.  Only weights quantised along K are supported."""
    if mx_axis not in (-2, 1):
        raise NotImplementedError("MXFP4 weights must be quantised along K (mx_axis = -2)")
    return B200MXValueLayout()


def make_default_matmul_mxfp4_w_scale_layout(mx_axis: int = -2, num_warps: int = 8):
    """Scale layout matching `make_default_matmul_mxfp4_w_layout` (layout.py:49-54 of the reference); `num_warps` matters
    only to the reference's Hopper layout."""
    if mx_axis not in (-2, 1):
        raise NotImplementedError("MXFP4 weights must be quantised along K (mx_axis = -2)")
    return B200MXScaleLayout()
