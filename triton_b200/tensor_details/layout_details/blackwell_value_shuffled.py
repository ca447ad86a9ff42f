"""BlackwellMX4ValueShuffledLayout: MXFP4 weight values pre-cut into tiles of `block_n` columns x `block_k` k values
(block_k / 2 packed bytes), every tile contiguous, tiles ordered [E][k tile][n tile]
(triton_kernels/tensor_details/layout_details/blackwell_value_shuffled.py:13-57, 203-261).

Storage: uint8 [E, K_tiles, N_tiles, block_n, block_k / 2]; byte (e, tk, tn, n, b) holds k = 2 * (tk * block_k / 2 + b)
in its low nibble and k + 1 in its high nibble of column tn * block_n + n.  The packed-K extent is padded to a multiple
of lcm(128, block_k / 2) bytes and N to a multiple of block_n, with zero bytes.  A caller that prepared weights for the
reference with `allow_blackwell_value_shuffle=True` holds this format; `convert_layout` brings it to the B200 layouts.
One-time weight preparation, torch ops on the tensor's device."""
import math
from dataclasses import dataclass

import torch

from .base import Layout, LayoutTransformation
from .strided import repack


@dataclass(frozen=True)
class BlackwellMX4ValueShuffledLayout(Layout):
    block_k: int = 128
    block_n: int = 256

    @property
    def name(self):
        return "BLACKWELL_MX4_VALUE_SHUFFLED"

    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        return BlackwellMX4ValueShuffledTransformation(list(shape), is_fp4, self.block_k, self.block_n)

    def swizzle_block_shape(self, block_shape):
        if len(block_shape) != 3:
            raise ValueError(f"Expected 3D block_shape, got {len(block_shape)}D: {block_shape}")
        _, block_k, block_n = block_shape
        if block_k != self.block_k:
            raise ValueError(f"block_k={block_k} does not match layout block_k={self.block_k}")
        return [1, 1, 1, block_n, block_k]


@dataclass(frozen=True)
class BlackwellMX4ValueShuffledTransformation(LayoutTransformation):
    block_k: int = 128
    block_n: int = 256

    def _tiling(self):
        if not self.is_fp4:
            raise ValueError("BlackwellMX4ValueShuffledLayout only supports fp4 values")
        *lead, K, N = self.shape
        if K % 2 or N % 2:
            raise ValueError(f"FP4 packing needs even K and N, got K={K}, N={N}")
        kb, tkb = K // 2, self.block_k // 2                 # packed bytes along K, per tile
        quantum = math.lcm(128, tkb)
        kb_pad = -(-kb // quantum) * quantum
        n_pad = -(-N // self.block_n) * self.block_n
        return math.prod(lead), kb, N, tkb, kb_pad, n_pad

    @property
    def storage_shape(self):
        E, kb, N, tkb, kb_pad, n_pad = self._tiling()
        return [E, kb_pad // tkb, n_pad // self.block_n, self.block_n, tkb]

    def swizzle_data(self, data):
        E, kb, N, tkb, kb_pad, n_pad = self._tiling()
        q = repack(data.reshape(E, 2 * kb, N // 2), -1, -2, True)                       # [E, K/2, N], packed along K
        padded = torch.zeros((E, kb_pad, n_pad), dtype=q.dtype, device=q.device)
        padded[:, :kb, :N] = q
        tiles = padded.reshape(E, kb_pad // tkb, tkb, n_pad // self.block_n, self.block_n)
        return self._validate_storage_shape(tiles.permute(0, 1, 3, 4, 2).contiguous())  # [E, tk, tn, n, byte]

    def unswizzle_data(self, data):
        E, kb, N, tkb, kb_pad, n_pad = self._tiling()
        q = data.permute(0, 1, 4, 2, 3).reshape(E, kb_pad, n_pad)[:, :kb, :N]
        out = repack(q.contiguous(), -2, -1, True)                                      # [E, K, N/2], packed along N
        return out.reshape(*self.shape[:-1], N // 2).contiguous()
