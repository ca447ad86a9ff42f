"""The weight layouts the tcgen05 grouped GEMM streams: tiles of 128 n x 128 k, ordered
[E][n_tile][k_tile], each tile contiguous so that one bulk copy fetches it.

* B200MXValueLayout: a tile is 128 rows x 64 bytes; every 32-bit word holds k = 8j .. 8j+7 with the
  nibbles reordered (k0,k2,k4,k6,k1,k3,k5,k7), which lets the kernel peel bf16 pairs with one mask.
* B200MXScaleLayout: a tile is 128 rows x 4 e8m0 bytes.

* B200BlockScaledValueLayout / B200BlockScaledScaleLayout: the same 128 x 128 tiles ordered
  [E][k_tile][n_block] for the block-scaled kernel (tcgen05.mma.kind::mxf8f6f4): plain packed e2m1 rows of 64
  bytes that the TMA unit expands on its way into shared memory, and scale tiles in the 128 x 4 packed-block order
  [r % 32][r / 32][group] that tcgen05.cp moves into tensor memory.

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


# ---- layouts of the block-scaled kernel ------------------------------------------------------------------------
@dataclass(frozen=True)
class B200BlockScaledValueLayout(Layout):

    @property
    def name(self):
        return "B200_BLOCK_SCALED_VALUE"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        assert is_fp4, "B200BlockScaledValueLayout holds e2m1 values"
        return B200BlockScaledValueLayoutTransformation(list(shape), is_fp4)


@dataclass(frozen=True)
class B200BlockScaledScaleLayout(Layout):

    @property
    def name(self):
        return "B200_BLOCK_SCALED_SCALE"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return B200BlockScaledScaleLayoutTransformation(list(shape), is_fp4)


@dataclass(frozen=True)
class B200BlockScaledValueLayoutTransformation(B200MXValueLayoutTransformation):
    """Same sizes as B200MXValueLayoutTransformation; tiles ordered [E][k_tile][n_block], nibbles in natural order."""

    def swizzle_data(self, data):
        from .strided import repack
        E, K, N, NT, KT = _tiles(self.shape)
        assert K % 32 == 0, "MXFP4 weights need K % 32 == 0"
        q = repack(data.reshape(E, K, N // 2), -1, -2, True).transpose(-1, -2).contiguous()     # [E, N, K/2]
        out = torch.empty(self.storage_shape, dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_to_b200mx(_lib.ptr(q), N * (K // 2), K // 2, None, 0, 0, 0, E, K, N,
                                                   _lib.ptr(out), None, _lib.stream()), "moe_weight_layout_to_b200mx")
        return out

    def unswizzle_data(self, data):
        from .strided import repack
        E, K, N, NT, KT = _tiles(self.shape)
        q = torch.empty((E, N, K // 2), dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_from_b200mx(_lib.ptr(data), None, E, K, N, _lib.ptr(q), None, _lib.stream()),
                   "moe_weight_layout_from_b200mx")
        out = repack(q.transpose(-1, -2), -2, -1, True)                 # [E, K, N/2]
        return out.reshape(*self.shape[:-1], N // 2).contiguous()


@dataclass(frozen=True)
class B200BlockScaledScaleLayoutTransformation(B200MXScaleLayoutTransformation):

    def swizzle_data(self, data):
        *lead, KG, N = self.shape
        E, K, N, NT, KT = _tiles([*lead, KG * 32, N])
        s = data.reshape(E, KG, N).contiguous()
        out = torch.empty(self.storage_shape, dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_to_b200mx(None, 0, 0, _lib.ptr(s), KG * N, N, 1, E, K, N, None, _lib.ptr(out),
                                                   _lib.stream()), "moe_weight_layout_to_b200mx")
        return out

    def unswizzle_data(self, data):
        *lead, KG, N = self.shape
        E, K, N, NT, KT = _tiles([*lead, KG * 32, N])
        s = torch.empty((E, N, KG), dtype=torch.uint8, device=data.device)
        lib = _lib.load()
        _lib.check(lib.moe_weight_layout_from_b200mx(None, _lib.ptr(data), E, K, N, None, _lib.ptr(s), _lib.stream()),
                   "moe_weight_layout_from_b200mx")
        return s.transpose(-1, -2).contiguous().reshape(*lead, KG, N)
