"""Ragged-segment metadata: per-slice offsets and the packed block schedules for row blocks of
16/32/64/128 (triton_kernels/tensor_details/ragged_tensor.py:12-94, 183-210, 348-381)."""
from dataclasses import dataclass

import torch

from .. import _lib


@dataclass
class RaggedTensorMetadata:
    """slice_sizes [E]; slice_offs [E+1] = exclusive cumsum; block_offs_data [4, E+1] = exclusive cumsum of
    ceil(slice_sizes / (16 << b)); block_schedule_data [4, max_n_blocks] with entries
    (block_in_slice << 16) | slice_id, padded with -1."""
    slice_sizes: torch.Tensor
    slice_offs: torch.Tensor
    block_offs_data: torch.Tensor
    block_schedule_data: torch.Tensor
    expected_slice_size: int | None = None
    slice_sizes_divisibility: int = None

    def __post_init__(self):
        assert self.block_offs_data.shape[0] == len(RaggedTensorMetadata.block_sizes())
        assert self.block_schedule_data.shape[0] == len(RaggedTensorMetadata.block_sizes())
        assert self.block_offs_data.dtype == torch.int32
        assert self.block_schedule_data.dtype == torch.int32
        if self.slice_sizes is not None:
            assert self.slice_sizes.dtype == torch.int32
        if self.slice_offs is not None:
            assert self.slice_offs.dtype == torch.int32

    @property
    def n_slices(self):
        return self.slice_sizes.shape[0]

    def block_offs(self, block_size):
        return self.block_offs_data[RaggedTensorMetadata.block_sizes().index(block_size)]

    def block_schedule(self, block_size):
        return self.block_schedule_data[RaggedTensorMetadata.block_sizes().index(block_size)]

    @staticmethod
    def n_blocks(n_slices, n_total_rows, block_size):
        if n_total_rows <= n_slices:
            return n_total_rows
        return n_slices - 1 - ((n_slices - n_total_rows - 1) // block_size)

    @staticmethod
    def max_n_blocks(n_slices, n_total_rows):
        return RaggedTensorMetadata.n_blocks(n_slices, n_total_rows, min(RaggedTensorMetadata.block_sizes()))

    @staticmethod
    def block_sizes_log2():
        return range(4, 8)

    @staticmethod
    def block_sizes():
        return [2**x for x in RaggedTensorMetadata.block_sizes_log2()]


def ragged_metadata_fields(metadata, block_size):
    return (metadata.slice_sizes, metadata.slice_offs, metadata.block_offs(block_size),
            metadata.block_schedule(block_size), metadata.expected_slice_size, metadata.slice_sizes_divisibility or 1)


def _empty_aligned(shape, device, pad=512):
    cols = (shape[-1] + pad - 1) // pad * pad
    full = torch.empty((*shape[:-1], max(cols, pad)), dtype=torch.int32, device=device)
    return full[..., : shape[-1]]


def make_ragged_tensor_metadata(slice_sizes, n_total_rows):
    assert slice_sizes.ndim == 1
    lib = _lib.load()
    E = slice_sizes.shape[0]
    dev = slice_sizes.device
    slice_sizes = slice_sizes.to(torch.int32).contiguous()
    mnb = RaggedTensorMetadata.max_n_blocks(E, n_total_rows)
    offs = _empty_aligned((5, E + 1), dev)
    sched = _empty_aligned((4, mnb), dev)
    slice_offs, block_offs = offs[0], offs[1:]
    _lib.check(lib.moe_ragged_metadata(_lib.ptr(slice_sizes), E, _lib.ptr(slice_offs), _lib.ptr(block_offs),
                                       block_offs.stride(0), _lib.ptr(sched), sched.stride(0), mnb, _lib.stream()),
               "moe_ragged_metadata")
    return RaggedTensorMetadata(slice_sizes, slice_offs, block_offs, sched)


def remap_ragged_tensor_metadata(src: RaggedTensorMetadata, slice_map: torch.Tensor) -> RaggedTensorMetadata:
    """Metadata of the ragged tensor made of the slices with ``slice_map[e] != -1`` (in order), slice ids
    rewritten through `slice_map`, offsets kept global."""
    assert slice_map.ndim == 1 and slice_map.shape[0] == src.slice_sizes.shape[0]
    lib = _lib.load()
    E = src.slice_sizes.shape[0]
    dev = src.slice_sizes.device
    slice_map = slice_map.to(torch.int32).contiguous()
    mnb = src.block_schedule_data.shape[-1]
    sizes = torch.empty_like(src.slice_sizes)
    offs = _empty_aligned((5, E + 1), dev)
    sched = _empty_aligned((4, mnb), dev)
    slice_offs, block_offs = offs[0], offs[1:]
    assert block_offs.stride(0) == src.block_offs_data.stride(0) and sched.stride(0) == src.block_schedule_data.stride(0)
    _lib.check(lib.moe_ragged_metadata_remap(
        _lib.ptr(src.slice_sizes), _lib.ptr(src.slice_offs), _lib.ptr(src.block_offs_data), src.block_offs_data.stride(0),
        _lib.ptr(src.block_schedule_data), src.block_schedule_data.stride(0), mnb, _lib.ptr(slice_map), E,
        _lib.ptr(sizes), _lib.ptr(slice_offs), _lib.ptr(block_offs), _lib.ptr(sched), _lib.stream()),
        "moe_ragged_metadata_remap")
    return RaggedTensorMetadata(sizes, slice_offs, block_offs, sched)
