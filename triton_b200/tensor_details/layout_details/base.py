"""Layout / LayoutTransformation interfaces (triton_kernels/tensor_details/layout_details/base.py)."""
from abc import ABC, abstractmethod
from dataclasses import dataclass


@dataclass(frozen=True)
class LayoutTransformation(ABC):
    shape: list
    is_fp4: bool

    @property
    def storage_shape(self) -> list:
        raise NotImplementedError

    def _validate_storage_shape(self, data):
        assert list(data.shape) == self.storage_shape, (list(data.shape), self.storage_shape)
        return data

    @abstractmethod
    def swizzle_data(self, data):
        """canonical (row-major, packed along the last axis) -> this layout"""

    @abstractmethod
    def unswizzle_data(self, data):
        """this layout -> canonical"""


@dataclass(frozen=True)
class Layout(ABC):

    def can_preserve_storage_as(self, other: "Layout", rank: int) -> bool:
        return self == other

    def storage_shape(self, shape, is_fp4: bool):
        return self.make_transformation(shape, is_fp4).storage_shape

    @abstractmethod
    def make_transformation(self, shape, is_fp4: bool) -> LayoutTransformation:
        pass

    def swizzle_block_shape(self, block_shape):
        return block_shape
