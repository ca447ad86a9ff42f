"""Expert weights on disk, already in the layouts the kernels stream.

Re-laying out MXFP4 weights (nibble reorder, tiling, scale blocks) is a pure function of what `downcast_to_mxfp`
returns, so it is done once and the result cached: one file per layer holds the tiled values and scales of fc1 and
fc2 (optionally the block-scaled copies too), the biases and the activation parameters.  Loading is a read into
pinned memory and one host-to-device copy per tensor; nothing is recomputed.

File format (little endian):
    bytes 0..7     magic  b"MOEB200W"
    bytes 8..11    uint32 version (1)
    bytes 12..15   uint32 length L of the JSON header
    bytes 16..16+L JSON: {"alpha", "limit", "tensors": {name: {"dtype", "shape", "layout", "logical_shape", "logical_dtype",
                          "offset", "nbytes"}}}; offsets are absolute and multiples of 4096
    then the raw tensors.

`from_block_checkpoint` reads the other on-disk form of MXFP4 experts, the one model checkpoints use: values as
`blocks` uint8 [E, N, K/32, 16] (16 bytes = 32 e2m1 values of one group along K, low nibble first) and `scales` uint8
[E, N, K/32] -- that is the canonical K-packed form (numerics_details/mxfp.py:25-88 of the reference with axis = K)
under another shape, so it converts to the tiled layouts without touching a value.
"""
import json
import struct
from pathlib import Path

import numpy as np
import torch

from .moe import MoeLayerWeights
from .tensor import FP4, Storage, Tensor, convert_layout, torch_dtype_to_dtype, wrap_torch_tensor
from .tensor_details.layout import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout, B200MXScaleLayout,
                                    B200MXValueLayout)

MAGIC = b"MOEB200W"
VERSION = 1
ALIGN = 4096

_LAYOUTS = {"B200_MX_VALUE": B200MXValueLayout, "B200_MX_SCALE": B200MXScaleLayout,
            "B200_BLOCK_SCALED_VALUE": B200BlockScaledValueLayout, "B200_BLOCK_SCALED_SCALE": B200BlockScaledScaleLayout}
_NP = {"uint8": np.uint8, "bfloat16": np.uint16, "float16": np.float16, "float32": np.float32}
_FIELDS = ("w1", "w1_scale", "b1", "w2", "w2_scale", "b2", "w1_bs", "w1_bs_scale", "w2_bs", "w2_bs_scale")


def _entry(name, obj):
    if isinstance(obj, Tensor):
        data = obj.storage.data
        lay = obj.storage.layout.name
        if lay not in _LAYOUTS:
            raise ValueError(f"{name}: layout {lay} is not one of the tiled B200 layouts; convert_layout first")
        logical = {"layout": lay, "logical_shape": [int(v) for v in obj.shape], "logical_dtype": "fp4" if obj.dtype == FP4 else "uint8"}
    else:
        data, logical = obj, {"layout": None, "logical_shape": None, "logical_dtype": None}
    data = data.detach().contiguous().cpu()
    dt = str(data.dtype).split(".")[-1]
    if dt not in _NP:
        raise ValueError(f"{name}: dtype {dt} is not supported by the weight file")
    raw = data.view(torch.uint16).numpy() if data.dtype == torch.bfloat16 else data.numpy()
    return {"dtype": dt, "shape": [int(v) for v in data.shape], **logical}, raw


def save_layer_weights(path, lw: MoeLayerWeights):
    """Write `lw` (tiled layouts, biases, activation parameters) to `path`."""
    entries, blobs = {}, {}
    for name in _FIELDS:
        obj = getattr(lw, name, None)
        if obj is None:
            continue
        entries[name], blobs[name] = _entry(name, obj)
    header = {"alpha": lw.alpha, "limit": lw.limit, "tensors": entries}
    # offsets depend on the header length, which depends on the offsets' digits: reserve a fixed-width header block
    pos = ALIGN * 4
    for name in entries:
        entries[name]["offset"] = pos
        entries[name]["nbytes"] = int(blobs[name].nbytes)
        pos = (pos + blobs[name].nbytes + ALIGN - 1) // ALIGN * ALIGN
    hj = json.dumps(header).encode()
    if 16 + len(hj) > ALIGN * 4:
        raise ValueError("weight file header too large")
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<II", VERSION, len(hj)) + hj)
        for name in entries:
            f.seek(entries[name]["offset"])
            f.write(blobs[name].tobytes())
        f.truncate(pos)
    return pos


def read_header(path):
    with open(path, "rb") as f:
        head = f.read(16)
        if len(head) < 16 or head[:8] != MAGIC:
            raise ValueError(f"{path}: not a MOEB200W weight file")
        version, n = struct.unpack("<II", head[8:16])
        if version != VERSION:
            raise ValueError(f"{path}: weight file version {version}, this reader knows {VERSION}")
        return json.loads(f.read(n).decode())


def load_layer_weights(path, device) -> MoeLayerWeights:
    """Read a file written by `save_layer_weights` onto `device` (memory-mapped read, pinned staging when the device is
    a GPU).  The tensors come back in the layouts they were saved in: no conversion runs."""
    header = read_header(path)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    dev = torch.device(device)
    out = {}
    for name, e in header["tensors"].items():
        raw = np.frombuffer(mm, dtype=_NP[e["dtype"]], count=int(np.prod(e["shape"])) if e["shape"] else 1, offset=e["offset"])
        t = torch.from_numpy(raw.reshape(e["shape"]).copy())
        if e["dtype"] == "bfloat16":
            t = t.view(torch.bfloat16)
        if dev.type == "cuda":
            t = t.pin_memory().to(dev, non_blocking=True)
        if e["layout"] is not None:
            dtype = FP4 if e["logical_dtype"] == "fp4" else torch_dtype_to_dtype(torch.uint8)
            t = Tensor(Storage(t, _LAYOUTS[e["layout"]]()), dtype=dtype, shape=list(e["logical_shape"]))
        out[name] = t
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    return MoeLayerWeights(out["w1"], out["w1_scale"], out["b1"], out["w2"], out["w2_scale"], out["b2"],
                           alpha=header["alpha"], limit=header["limit"], w1_bs=out.get("w1_bs"),
                           w1_bs_scale=out.get("w1_bs_scale"), w2_bs=out.get("w2_bs"), w2_bs_scale=out.get("w2_bs_scale"))


def tensors_from_blocks(blocks: torch.Tensor, scales: torch.Tensor, block_scaled=False):
    """Checkpoint form -> (values Tensor, scales Tensor) in the tiled B200 layouts.

    blocks uint8 [E, N, K/32, 16], scales uint8 [E, N, K/32] (the expert weight is W[e] of shape [K, N], quantised along
    K).  Both live on a CUDA device (the re-layout is a kernel of the library)."""
    assert blocks.dtype == torch.uint8 and scales.dtype == torch.uint8
    E, N, G, B = blocks.shape
    assert B == 16 and tuple(scales.shape) == (E, N, G), "expected blocks [E, N, K/32, 16] and scales [E, N, K/32]"
    q = blocks.reshape(E, N, G * 16).transpose(1, 2)        # [E, K/2, N] with K contiguous: the canonical K-packed form
    s = scales.transpose(1, 2)                              # [E, K/32, N]
    vl, sl = (B200BlockScaledValueLayout(), B200BlockScaledScaleLayout()) if block_scaled else (B200MXValueLayout(), B200MXScaleLayout())
    return convert_layout(wrap_torch_tensor(q, dtype=FP4), vl), convert_layout(wrap_torch_tensor(s), sl)


def from_block_checkpoint(w1_blocks, w1_scales, b1, w2_blocks, w2_scales, b2, alpha=1.702, limit=7.0, block_scaled=False):
    """A layer from checkpoint tensors: fc1 `*_blocks` [E, 2*d_ff, d_model/32, 16] (gate and linear rows interleaved, as
    the layer's SwiGLU expects), fc2 [E, d_model, d_ff/32, 16], biases [E, 2*d_ff] and [E, d_model]."""
    w1, s1 = tensors_from_blocks(w1_blocks, w1_scales)
    w2, s2 = tensors_from_blocks(w2_blocks, w2_scales)
    lw = MoeLayerWeights(w1, s1, b1, w2, s2, b2, alpha=alpha, limit=limit)
    if block_scaled:
        lw.w1_bs, lw.w1_bs_scale = tensors_from_blocks(w1_blocks, w1_scales, True)
        lw.w2_bs, lw.w2_bs_scale = tensors_from_blocks(w2_blocks, w2_scales, True)
    return lw
