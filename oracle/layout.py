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


def swizzle_mx4_value_shuffled_oracle(w: torch.Tensor, block_k: int = 128, block_n: int = 256) -> torch.Tensor:
    """Canonical [E, K, N/2] (packed along N) -> [E, K_tiles, N_tiles, block_n, block_k/2] packed along K: tile
    (tk, tn) holds columns tn*block_n.. and packed-K bytes tk*block_k/2.., rows = columns of the weight
    (``blackwell_value_shuffled.py:138-166``); packed K padded to lcm(128, block_k/2), N to block_n, zero fill.
    Element-wise definition (slow, small cases only)."""
    import math
    r = repack_fp4_oracle(w, -1, -2)                               # [E, K/2, N]
    E, kb, N = r.shape
    tkb = block_k // 2
    quantum = math.lcm(128, tkb)
    kbp = -(-kb // quantum) * quantum
    npad = -(-N // block_n) * block_n
    out = torch.zeros(E, kbp // tkb, npad // block_n, block_n, tkb, dtype=torch.uint8)
    for e in range(E):
        for b in range(kb):
            for n in range(N):
                out[e, b // tkb, n // block_n, n % block_n, b % tkb] = r[e, b, n]
    return out


def swizzle_act_mx_scale_oracle(s: torch.Tensor, slice_sizes=None) -> torch.Tensor:
    """Activation scales [M, K/32] -> [1, M_pad/128, K_pad/4, 2, 256] in blocks of 128 rows x 4 groups stored
    [32 lanes][4 quads][4 k] (``blackwell_scale.py:104-121``); with ``slice_sizes`` every slice of rows starts at a new
    block of 128 rows (``:68-80``, the reference pads with a GPU kernel: this ragged form is defined here and unpinned)."""
    M, K = s.shape
    Kp = (K + 7) // 8 * 8
    if slice_sizes is None:
        Mp = (M + 127) // 128 * 128
        rows = list(range(M))
    else:
        from .routing import n_blocks
        Mp = 128 * n_blocks(len(slice_sizes), M, 128)
        rows, off, blk = [-1] * M, 0, 0
        for sz in [int(v) for v in slice_sizes]:
            for j in range(sz):
                rows[off + j] = blk * 128 + j
            off += sz
            blk += (sz + 127) // 128
    out = torch.zeros(Mp // 128, Kp // 4, 32, 4, 4, dtype=torch.uint8)
    for m in range(M):
        if rows[m] < 0:
            continue
        r = rows[m]
        for k in range(K):
            out[r // 128, k // 4, (r % 128) % 32, (r % 128) // 32, k % 4] = s[m, k]
    return out.reshape(1, Mp // 128, Kp // 4, 2, 256)
