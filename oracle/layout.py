"""CPU oracle for the Blackwell weight layouts (TEST INFRASTRUCTURE ONLY).

Follows ``tensor_details/layout_details/blackwell_scale.py:146-209`` (scale tiles of
128 N-rows x 4 K-groups, stored ``[32 lanes][4 quads][4 k]``), ``blackwell_value.py:35-70``
(K-packed column-major values with the packed-K extent padded to 128 bytes) and
``torch_utils.py:44-91`` (nibble re-packing between axes).
"""
import torch
import torch.nn.functional as F


def swizzle_mx_scale_bw_oracle(s: torch.Tensor) -> torch.Tensor:
    """[..., K/32, N] uint8 -> [1, B*Npad/128, Kpad/4, 2, 256]; K padded to 8, N to 128, zero fill."""
    *lead, K, N = s.shape
    B = 1
    for d in lead:
        B *= d
    Kp, Np = (K + 7) // 8 * 8, (N + 127) // 128 * 128
    d = F.pad(s.reshape(B, K, N), (0, Np - N, 0, Kp - K))
    d = d.transpose(-1, -2).contiguous()                     # [B, Np, Kp]
    d = d.reshape(B, Np // 128, 4, 32, Kp // 4, 4)           # [b, nblk, quad, lane, kgrp, k]
    d = d.permute(0, 1, 4, 3, 2, 5).contiguous()             # [b, nblk, kgrp, lane, quad, k]
    return d.reshape(1, B * Np // 128, Kp // 4, 2, 256)


def unswizzle_mx_scale_bw_oracle(d: torch.Tensor, shape) -> torch.Tensor:
    *lead, K, N = shape
    B = 1
    for x in lead:
        B *= x
    Kp, Np = (K + 7) // 8 * 8, (N + 127) // 128 * 128
    d = d.reshape(B, Np // 128, Kp // 4, 32, 4, 4).permute(0, 1, 4, 3, 2, 5)
    d = d.reshape(*lead, Np, Kp).transpose(-1, -2)
    return d[..., :K, :N].contiguous()


def repack_fp4_oracle(data: torch.Tensor, old_dim: int, new_dim: int) -> torch.Tensor:
    """Move the nibble-packing axis of an e2m1x2 byte tensor from `old_dim` to `new_dim`."""
    old_dim %= data.ndim
    new_dim %= data.ndim
    if old_dim == new_dim:
        return data.clone()
    lo, hi = data & 0xF, data >> 4
    shp = list(data.shape)
    shp[old_dim] *= 2
    nib = torch.stack([lo, hi], dim=old_dim + 1).reshape(shp)     # unpacked nibbles
    idx_e = [slice(None)] * data.ndim
    idx_o = [slice(None)] * data.ndim
    idx_e[new_dim] = slice(0, None, 2)
    idx_o[new_dim] = slice(1, None, 2)
    return nib[tuple(idx_e)] | (nib[tuple(idx_o)] << 4)


def swizzle_mx_value_bw_oracle(w: torch.Tensor) -> torch.Tensor:
    """Canonical [..., K, N/2] (packed along N, row-major) -> [..., pad128(K/2), N] packed along K,
    with the packed-K axis contiguous (column-major)."""
    r = repack_fp4_oracle(w, -1, -2)                               # [..., K/2, N]
    kp = r.shape[-2]
    pad = (-kp) % 128
    out = torch.zeros(*r.shape[:-2], kp + pad, r.shape[-1], dtype=torch.uint8)
    out[..., :kp, :] = r
    return out


def unswizzle_mx_value_bw_oracle(d: torch.Tensor, shape) -> torch.Tensor:
    K = shape[-2]
    return repack_fp4_oracle(d[..., : K // 2, :], -2, -1)
