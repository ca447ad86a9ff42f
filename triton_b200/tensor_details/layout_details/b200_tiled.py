"""The weight layouts the tcgen05 grouped GEMM streams: tiles of 128 n x 128 k, ordered
[E][n_tile][k_tile], each tile contiguous so that one bulk copy fetches it.

* B200MXValueLayout: a tile is 128 rows x 64 bytes; every 32-bit word holds k = 8j .. 8j+7 with the
  nibbles reordered (k0,k2,k4,k6,k1,k3,k5,k7), which lets the kernel peel bf16 pairs with one mask.
* B200MXScaleLayout: a tile is 128 rows x 4 e8m0 bytes.

They play the role of BlackwellMX4ValueShuffledLayout / BlackwellMXScaleLayout of the reference
(triton_kernels/tensor_details/layout_details/blackwell_value_shuffled.py:13-57, blackwell_scale.py:16-30):
`convert_layout(w, B200MXValueLayout())` is done once when weights are loaded.  Values and scales are
converted by one CUDA kernel pair (csrc/layout.cu); storage is a flat uint8 buffer.
"""
from dataclasses import dataclass

import torch

from ... import _lib
from .base import Layout, LayoutTransformation

TILE = 128


def _tiles(shape):
    *lead, K, N = shape
    E = 1
    for d in lead:
        E *= d
    return E, K, N, (N + TILE - 1) // TILE, (K + TILE - 1) // TILE


@dataclass(frozen=True)
class B200MXValueLayout(Layout):

    @property
    def name(self):
        return "B200_MX_VALUE"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        assert is_fp4, "B200MXValueLayout holds e2m1 values"
        return B200MXValueLayoutTransformation(list(shape), is_fp4)


@dataclass(frozen=True)
class B200MXScaleLayout(Layout):

    @property
    def name(self):
        return "B200_MX_SCALE"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return B200MXScaleLayoutTransformation(list(shape), is_fp4)


@dataclass(frozen=True)
class B200MXValueLayoutTransformation(LayoutTransformation):
    """`shape` is the logical [..., K, N]; canonical data is [..., K, N/2] packed along N."""

    @property
    def storage_shape(self):
        E, K, N, NT, KT = _tiles(self.shape)
        return [E * NT * KT * TILE * (TILE // 2)]

    def swizzle_data(self, data):
        from .strided import repack
        E, K, N, NT, KT = _tiles(self.shape)
        assert K % 32 == 0, "MXFP4 weights need K % 32 == 0"
        q = repack(data.reshape(E, K, N // 2), -1, -2, True)            # [E, K/2, N]
        q = q.transpose(-1, -2).contiguous()                            # [E, N, K/2], K contiguous
        out = torch.empty(self.storage_shape, dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_to_b200(_lib.ptr(q), N * (K // 2), K // 2, None, 0, 0, 0, E, K, N,
                                                 _lib.ptr(out), None, _lib.stream()), "moe_weight_layout_to_b200")
        return out

    def unswizzle_data(self, data):
        from .strided import repack
        E, K, N, NT, KT = _tiles(self.shape)
        q = torch.empty((E, N, K // 2), dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_from_b200(_lib.ptr(data), None, E, K, N, _lib.ptr(q), None, _lib.stream()),
                   "moe_weight_layout_from_b200")
        q = q.transpose(-1, -2)                                         # [E, K/2, N]
        out = repack(q, -2, -1, True)                                   # [E, K, N/2]
        return out.reshape(*self.shape[:-1], N // 2).contiguous()


@dataclass(frozen=True)
class B200MXScaleLayoutTransformation(LayoutTransformation):
    """`shape` is the logical scale shape [..., K/32, N]; canonical data has the same shape, row-major."""

    @property
    def storage_shape(self):
        *lead, KG, N = self.shape
        E, K, N, NT, KT = _tiles([*lead, KG * 32, N])
        return [E * NT * KT * TILE * 4]

    def swizzle_data(self, data):
        *lead, KG, N = self.shape
        E, K, N, NT, KT = _tiles([*lead, KG * 32, N])
        s = data.reshape(E, KG, N).contiguous()
        out = torch.empty(self.storage_shape, dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_to_b200(None, 0, 0, _lib.ptr(s), KG * N, N, 1, E, K, N, None, _lib.ptr(out),
                                                 _lib.stream()), "moe_weight_layout_to_b200")
        return out

    def unswizzle_data(self, data):
        *lead, KG, N = self.shape
        E, K, N, NT, KT = _tiles([*lead, KG * 32, N])
        s = torch.empty((E, N, KG), dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_from_b200(None, _lib.ptr(data), E, K, N, None, _lib.ptr(s), _lib.stream()),
                   "moe_weight_layout_from_b200")
        return s.transpose(-1, -2).contiguous().reshape(*lead, KG, N)
