"""BlackwellMXScaleLayout: e8m0 scales in tiles of 128 N-rows x 4 K-groups stored
[32 lanes][4 quads][4 k], storage shape [1, B*Npad/128, Kpad/4, 2, 256]
(triton_kernels/tensor_details/layout_details/blackwell_scale.py:16-30, 146-209).
One-time weight preparation, torch ops on the tensor's device."""
import math
from dataclasses import dataclass

import torch.nn.functional as F

from .base import Layout, LayoutTransformation


@dataclass(frozen=True)
class BlackwellMXScaleLayout(Layout):

    @property
    def name(self):
        return "BLACKWELL_SCALE"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return BlackwellMXScaleLayoutTransformation(list(shape), is_fp4)

    def swizzle_block_shape(self, block_shape):
        K, N = block_shape
        assert K % 4 == 0 and N % 128 == 0
        return [1, N // 128, K // 4, 2, 256]


@dataclass(frozen=True)
class BlackwellMXScaleLayoutTransformation(LayoutTransformation):

    def _dims(self):
        *lead, K, N = self.shape
        return lead, K, N, math.prod(lead), (K + 7) // 8 * 8, (N + 127) // 128 * 128

    @property
    def storage_shape(self):
        _, _, _, B, Kp, Np = self._dims()
        return [1, B * Np // 128, Kp // 4, 2, 256]

    def swizzle_data(self, data):
        _, K, N, B, Kp, Np = self._dims()
        d = F.pad(data.reshape(B, K, N), (0, Np - N, 0, Kp - K))
        d = d.transpose(-1, -2).contiguous().reshape(B, Np // 128, 4, 32, Kp // 4, 4)
        d = d.permute(0, 1, 4, 3, 2, 5).contiguous()
        return self._validate_storage_shape(d.view(*self.storage_shape))

    def unswizzle_data(self, data):
        lead, K, N, B, Kp, Np = self._dims()
        d = data.reshape(B, Np // 128, Kp // 4, 32, 4, 4).permute(0, 1, 4, 3, 2, 5)
        d = d.reshape(*lead, Np, Kp).transpose(-1, -2)
        return d[..., :K, :N].contiguous()
