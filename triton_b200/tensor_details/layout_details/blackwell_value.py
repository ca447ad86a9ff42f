"""BlackwellMXValueLayout: K-packed, K-contiguous ("column-major") e2m1 values with the packed-K
extent padded to a multiple of 128 bytes (triton_kernels/tensor_details/layout_details/blackwell_value.py:8-70).
One-time weight preparation, torch ops on the tensor's device."""
from dataclasses import dataclass

import torch

from .base import Layout, LayoutTransformation
from .strided import repack


@dataclass(frozen=True)
class BlackwellMXValueLayout(Layout):

    @property
    def name(self):
        return "BLACKWELL_MX_VALUE"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return BlackwellMXValueLayoutTransformation(list(shape), is_fp4)


def _strides_major_dim_m2(shape):
    n = len(shape)
    if n <= 1:
        return [1] * n
    order = [n - 2, n - 1] + list(range(n - 3, -1, -1))
    st = [0] * n
    st[order[0]] = 1
    for prev, d in zip(order, order[1:]):
        st[d] = st[prev] * shape[prev]
    return st


@dataclass(frozen=True)
class BlackwellMXValueLayoutTransformation(LayoutTransformation):

    @property
    def storage_shape(self):
        *lead, K, N = self.shape
        kp = K // 2
        kp += -kp % 128
        return [*lead, kp, N]

    def swizzle_data(self, data):
        ss = self.storage_shape
        ret = torch.empty_strided(ss, _strides_major_dim_m2(ss), device=data.device, dtype=data.dtype).zero_()
        repack(data, -1, -2, self.is_fp4, out=ret[..., : self.shape[-2] // 2, :])
        return self._validate_storage_shape(ret)

    def unswizzle_data(self, data):
        data = data[..., : self.shape[-2] // 2, :]
        out_shape = list(self.shape)
        out_shape[-1] //= 2
        out = torch.empty(out_shape, device=data.device, dtype=data.dtype)
        repack(data, -2, -1, self.is_fp4, out=out)
        return out
