"""BlackwellMXScaleLayout: e8m0 scales in tiles of 128 N-rows x 4 K-groups stored
[32 lanes][4 quads][4 k], storage shape [1, B*Npad/128, Kpad/4, 2, 256]
(triton_kernels/tensor_details/layout_details/blackwell_scale.py:16-30, 146-209).
One-time weight preparation, torch ops on the tensor's device."""
import math
from dataclasses import dataclass

import torch
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


# ---- activation scales ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class BlackwellActMXScaleLayout(Layout):
    """e8m0 scales of microscaled ACTIVATIONS, [M, K/32] (or [B, M, K/32]), in the same 128-row x 4-group packed blocks
    [32 lanes][4 quads][4 k] as the weight scales, rows first
    (triton_kernels/tensor_details/layout_details/blackwell_scale.py:33-143).  With `ragged_metadata` every slice of rows
    is padded to whole blocks of 128 rows (slice e starts at block `block_offs(128)[e]`), so that a block never mixes the
    rows of two experts; the storage then has room for `n_blocks(n_slices, M, 128)` blocks."""
    ragged_metadata: object = None

    def can_preserve_storage_as(self, other: Layout, rank: int) -> bool:
        return isinstance(other, BlackwellActMXScaleLayout) and self.ragged_metadata is other.ragged_metadata

    @property
    def name(self):
        return "BLACKWELL_ACT_SCALE"

    def swizzle_block_shape(self, block_shape):
        N, K = block_shape
        assert K % 4 == 0 and N % 128 == 0
        return [1, N // 128, K // 4, 2, 256]

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return BlackwellActMXScaleLayoutTransformation(list(shape), is_fp4, self.ragged_metadata)


@dataclass(frozen=True)
class BlackwellActMXScaleLayoutTransformation(LayoutTransformation):
    ragged_metadata: object = None

    def _dims(self):
        if len(self.shape) == 2:
            B, (M, K) = 1, self.shape
        else:
            B, M, K = self.shape
        ragged = self.ragged_metadata is not None and len(self.shape) == 2
        if ragged:
            md = self.ragged_metadata
            m_pad = 128 * md.n_blocks(md.slice_sizes.shape[0], M, 128)
        else:
            m_pad = (M + 127) // 128 * 128
        return B, M, K, m_pad, (K + 7) // 8 * 8, ragged

    @property
    def storage_shape(self):
        B, M, K, m_pad, k_pad, _ = self._dims()
        return [1, B * m_pad // 128, k_pad // 4, 2, 256]

    def _padded_rows(self, M, device):
        """Destination row of every source row in the block-padded arrangement (-1: the row is padding of the input)."""
        md = self.ragged_metadata
        offs = md.slice_offs.to(device=device, dtype=torch.int64)               # [E + 1]
        blk = md.block_offs(128).to(device=device, dtype=torch.int64)           # [E + 1]
        m = torch.arange(M, device=device)
        e = torch.searchsorted(offs, m, right=True) - 1
        valid = (m < offs[-1]) & (e >= 0)
        e = e.clamp(0, offs.numel() - 2)
        return torch.where(valid, blk[e] * 128 + (m - offs[e]), torch.full_like(m, -1))

    def swizzle_data(self, data):
        B, M, K, m_pad, k_pad, ragged = self._dims()
        if ragged:
            dst = self._padded_rows(M, data.device)
            d = torch.zeros((1, m_pad, k_pad), dtype=data.dtype, device=data.device)
            keep = dst >= 0
            d[0, dst[keep], :K] = data[keep]
        else:
            d = F.pad(data.reshape(B, M, K), (0, k_pad - K, 0, m_pad - M))
        d = d.reshape(B, m_pad // 128, 4, 32, k_pad // 4, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
        return self._validate_storage_shape(d.view(*self.storage_shape))

    def unswizzle_data(self, data):
        B, M, K, m_pad, k_pad, ragged = self._dims()
        d = data.reshape(B, m_pad // 128, k_pad // 4, 32, 4, 4).permute(0, 1, 4, 3, 2, 5).reshape(B, m_pad, k_pad)
        if ragged:
            dst = self._padded_rows(M, data.device)
            out = torch.zeros((M, K), dtype=data.dtype, device=data.device)
            keep = dst >= 0
            out[keep] = d[0, dst[keep], :K]
            return out
        d = d[:, :M, :K]
        return (d[0] if len(self.shape) == 2 else d).contiguous()
