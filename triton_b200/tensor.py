"""Typed tensor wrapper (logical FP4 / BIT shapes over packed storage), layouts and the routing
metadata constructors (triton_kernels/tensor.py:18-313)."""
from dataclasses import dataclass

import torch

from .tensor_details import bitmatrix as bitmatrix_details
from .tensor_details import ragged_tensor as ragged_tensor_details
from .tensor_details.bitmatrix import BitmatrixMetadata  # noqa: F401
from .tensor_details.dtype import (BF16, BIT, FP4, FP8_E4M3FN, FP8_E4M3FNUZ, FP8_E5M2, FP16, FP32, FP64,  # noqa: F401
                                   INT16, INT32, INT64, UINT8, DataType, FloatType, IntegerType)
from .tensor_details.layout import Layout, StridedLayout
from .tensor_details.ragged_tensor import RaggedTensorMetadata


@dataclass
class Storage:
    data: torch.Tensor
    layout: Layout

    @property
    def device(self):
        return self.data.device


@dataclass
class Tensor:
    storage: Storage
    dtype: IntegerType | FloatType
    shape: list | None = None
    shape_max: list | None = None

    def __post_init__(self):
        assert isinstance(self.storage, Storage)
        if self.dtype.bitwidth < 8 and self.shape is None:
            raise ValueError("shape must be provided for sub-byte types")
        if self.shape is None:
            self.shape = list(self.storage.data.shape)
        self.shape = list(self.shape)
        is_int = lambda s: isinstance(s, int)
        is_item = lambda s: hasattr(s, "numel") and s.numel() == 1
        assert all(is_int(s) or is_item(s) for s in self.shape)
        if self.shape_max is None:
            self.shape_max = [None] * len(self.shape)
        self.shape_max = list(self.shape_max)
        for i, (s, smax) in enumerate(zip(self.shape, self.shape_max)):
            if smax is not None and not is_int(smax):
                raise ValueError(f"shape_max[{i}] must be `int` or `None`; got {type(smax)}")
            if smax is None:
                self.shape_max[i] = s
        assert all(map(is_int, self.shape_max))

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def device(self):
        return self.storage.device

    def stride(self, i=None):
        return self.storage.data.stride() if i is None else self.storage.data.stride(i)

    def data_ptr(self):
        return self.storage.data.data_ptr()

    def numel(self):
        return self.storage.data.numel()

    def element_size(self):
        return self.dtype.bitwidth // 8

    @property
    def data(self):
        return self.storage.data

    def dim(self):
        return self.ndim

    def size(self, i=None):
        return self.shape if i is None else self.shape[i]


make_bitmatrix_metadata = bitmatrix_details.make_bitmatrix_metadata
make_ragged_tensor_metadata = ragged_tensor_details.make_ragged_tensor_metadata
remap_ragged_tensor_metadata = ragged_tensor_details.remap_ragged_tensor_metadata


@dataclass
class RaggedTensor:
    """A collection of 2-D slices sharing a column count, stored as one (possibly padded) 2-D tensor."""
    slice_sizes: torch.Tensor
    data: torch.Tensor
    metadata: RaggedTensorMetadata


@dataclass
class SparseMatrix:
    indx: torch.Tensor
    vals: torch.Tensor
    mask: Tensor
    mask_metadata: BitmatrixMetadata | None = None      # computed here unless the producer already has it

    def __post_init__(self):
        if self.mask_metadata is None:
            self.mask_metadata = make_bitmatrix_metadata(self.indx, self.mask)


def dtype_to_torch_dtype(dtype) -> torch.dtype:
    if not isinstance(dtype, (IntegerType, FloatType)):
        return dtype
    return {FP4: torch.uint8, UINT8: torch.uint8, FP8_E4M3FN: torch.float8_e4m3fn,
            FP8_E4M3FNUZ: torch.float8_e4m3fnuz, FP8_E5M2: torch.float8_e5m2, BF16: torch.bfloat16,
            FP32: torch.float32, FP16: torch.float16, FP64: torch.float64, INT16: torch.int16,
            INT32: torch.int32, INT64: torch.int64}[dtype]


def torch_dtype_to_dtype(dtype):
    if isinstance(dtype, (IntegerType, FloatType)):
        return dtype
    name = str(dtype).split(".")[-1]
    table = {"uint8": UINT8, "float8_e4m3fn": FP8_E4M3FN, "float8_e4m3fnuz": FP8_E4M3FNUZ, "float8_e5m2": FP8_E5M2,
             "float16": FP16, "bfloat16": BF16, "float32": FP32, "float64": FP64, "int16": INT16, "int32": INT32,
             "int64": INT64, "uint32": IntegerType(32, False), "bool": IntegerType(8, False)}
    if name in table:
        return table[name]
    raise ValueError(f"Unknown dtype: {name}")


def wrap_torch_tensor(torch_tensor, dtype=None, shape=None, shape_max=None, layout=None):
    if dtype is None:
        dtype = torch_tensor.dtype
    dtype = torch_dtype_to_dtype(dtype)
    if shape is None:
        shape = list(torch_tensor.shape)
        if dtype == FP4:
            shape[torch_tensor.stride().index(1)] *= (8 * torch_tensor.dtype.itemsize) // dtype.bitwidth
    if shape_max is None:
        shape_max = [s if isinstance(s, int) else None for s in shape]
        shape_max = [m if m is not None else int(torch_tensor.shape[i]) for i, m in enumerate(shape_max)]
    if layout is None:
        major = torch_tensor.stride().index(1) if 1 in torch_tensor.stride() else -1
        layout = StridedLayout(major_dim=major - torch_tensor.ndim if major >= 0 else -1)
    return Tensor(Storage(torch_tensor, layout), dtype=dtype, shape=shape, shape_max=shape_max)


def convert_layout(tensor: Tensor, layout: Layout, **kwargs):
    """Re-encode `tensor` storage as `layout` (through the canonical row-major form).  Returns `tensor`
    unchanged when its storage already is a valid encoding of `layout`."""
    shape = list(tensor.shape)
    if not kwargs and tensor.storage.layout.can_preserve_storage_as(layout, len(shape)):
        return tensor
    is_fp4 = tensor.dtype == FP4
    canonical = tensor.storage.layout.make_transformation(shape, is_fp4).unswizzle_data(tensor.storage.data)
    new_data = layout.make_transformation(shape, is_fp4, **kwargs).swizzle_data(canonical)
    return Tensor(Storage(new_data, layout), shape=shape, dtype=tensor.dtype)


def empty(shape, dtype, device, layout=None, allow_implicit_conversion: bool = False):
    storage_dtype = torch.uint8 if dtype == FP4 else dtype_to_torch_dtype(dtype)
    initial = layout if isinstance(layout, StridedLayout) else StridedLayout()
    storage_shape = initial.storage_shape(list(shape), dtype == FP4)
    strides = [0] * len(storage_shape)
    running = 1
    for d in initial.order(len(shape)):
        strides[d] = running
        running *= storage_shape[d]
    data = torch.empty_strided(storage_shape, strides, device=device, dtype=storage_dtype)
    ret = wrap_torch_tensor(data, dtype=dtype, shape=shape, layout=initial)
    if allow_implicit_conversion:
        ret = convert_layout(ret, layout)
    return ret
