"""Strided (canonical) layout: only the unit-stride ("major") dimension is recorded
(triton_kernels/tensor_details/layout_details/strided.py:9-98, torch_utils.py:44-91).

The nibble re-packing between axes is a one-time weight-preparation step and runs as torch integer
ops on the tensor's device."""
from dataclasses import dataclass

import torch

from .base import Layout, LayoutTransformation


def repack(data: torch.Tensor, old_dim: int, new_dim: int, is_fp4: bool, out=None) -> torch.Tensor:
    """Move the e2m1x2 packing axis of a byte tensor from `old_dim` to `new_dim`."""
    old_dim %= data.ndim
    new_dim %= data.ndim
    if (not is_fp4) or old_dim == new_dim:
        if out is not None:
            out.copy_(data)
            return out
        return data
    lo, hi = data & 0xF, data >> 4
    shp = list(data.shape)
    shp[old_dim] *= 2
    nib = torch.stack([lo, hi], dim=old_dim + 1).reshape(shp)
    ev = [slice(None)] * data.ndim
    od = [slice(None)] * data.ndim
    ev[new_dim] = slice(0, None, 2)
    od[new_dim] = slice(1, None, 2)
    res = nib[tuple(ev)] | (nib[tuple(od)] << 4)
    if out is not None:
        out.copy_(res)
        return out
    return res


@dataclass(frozen=True)
class StridedLayout(Layout):
    major_dim: int = -1

    def __post_init__(self):
        if not isinstance(self.major_dim, int):
            raise TypeError(f"StridedLayout(major_dim=...) must be an int, got {type(self.major_dim)}")

    @property
    def name(self):
        return "STRIDED"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return StridedLayoutTransformation(list(shape), is_fp4, self.order(len(shape)))

    def can_preserve_storage_as(self, other: Layout, rank: int) -> bool:
        return isinstance(other, StridedLayout) and self.order(rank) == other.order(rank)

    def order(self, rank: int):
        """minor -> major dimension order: reversed(range(rank)) with `major_dim` swapped to the front."""
        if rank <= 0:
            return []
        if not (-rank <= self.major_dim < rank):
            raise ValueError(f"Invalid StridedLayout.major_dim={self.major_dim} for rank={rank}")
        major = self.major_dim % rank
        base = list(reversed(range(rank)))
        i = base.index(major)
        base[0], base[i] = base[i], base[0]
        return base


@dataclass(frozen=True)
class StridedLayoutTransformation(LayoutTransformation):
    order: list

    @property
    def storage_shape(self):
        shape = list(self.shape)
        if self.is_fp4:
            pd = self.order[0]
            if shape[pd] % 2:
                raise ValueError(f"FP4 packing dimension {pd} must have an even size, got {shape[pd]}")
            shape[pd] //= 2
        return shape

    def swizzle_data(self, data):
        r = len(self.shape)
        if r == 0:
            return self._validate_storage_shape(data)
        out_shape = self.storage_shape
        stride, s = [0] * r, 1
        for d in self.order:
            stride[d], s = s, s * out_shape[d]
        out = torch.empty_strided(out_shape, stride, dtype=data.dtype, device=data.device)
        repack(data, -1, self.order[0], self.is_fp4, out=out)
        return self._validate_storage_shape(out)

    def unswizzle_data(self, data):
        out_shape = list(self.shape)
        if self.is_fp4:
            out_shape[-1] //= 2
        ret = torch.empty(out_shape, dtype=data.dtype, device=data.device)
        repack(data, self.order[0], -1, self.is_fp4, out=ret)
        return ret
