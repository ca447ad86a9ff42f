"""FnSpecs: names a function fused into a kernel (triton_kernels/specialize.py:68-78).  The reference
inlines the named Triton function by rewriting kernel source; here the name selects a compiled
epilogue variant of the CUDA kernel ("swiglu" or the default identity)."""
from dataclasses import dataclass
from typing import Callable, Optional


@dataclass(frozen=True)
class FnSpecs:
    name: str
    fn: Optional[Callable]
    fn_arg_names: tuple = tuple()
    fn_arg_do_not_specialize: tuple = tuple()
    reduction_n: int = 1

    @staticmethod
    def default():
        return FnSpecs("dflt", None, tuple())
