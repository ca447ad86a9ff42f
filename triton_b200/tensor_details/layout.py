"""Layout catalogue and the per-device defaults (triton_kernels/tensor_details/layout.py:27-54).

On B200 the default MXFP4 weight layouts are the tile-contiguous ones the tcgen05 kernel streams; the
reference's Blackwell layouts are kept for interchange (`convert_layout` goes through the canonical
form, so any pair of layouts converts both ways)."""
from .layout_details.base import Layout
from .layout_details.strided import StridedLayout
from .layout_details.blackwell_scale import BlackwellMXScaleLayout
from .layout_details.blackwell_value import BlackwellMXValueLayout
from .layout_details.b200_tiled import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout, B200MXScaleLayout,
                                        B200MXValueLayout)

__all__ = ["Layout", "StridedLayout", "BlackwellMXScaleLayout", "BlackwellMXValueLayout", "B200MXValueLayout",
           "B200MXScaleLayout", "B200BlockScaledValueLayout", "B200BlockScaledScaleLayout", "make_default_matmul_mxfp4_w_layout", "make_default_matmul_mxfp4_w_scale_layout"]


def make_default_matmul_mxfp4_w_layout(mx_axis: int = -2, allow_blackwell_value_shuffle: bool = False,
                                       block_k: int = 128, block_n: int = 256):
    return B200MXValueLayout()


def make_default_matmul_mxfp4_w_scale_layout(mx_axis: int = -2, num_warps: int = 8):
    return B200MXScaleLayout()
