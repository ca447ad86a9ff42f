"""The C-ABI library loads without a GPU and exports every symbol that include/moe_b200.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "moe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for required in ("moe_topk_fwd", "moe_bitmatrix_metadata", "moe_ragged_metadata", "moe_ragged_metadata_remap",
                     "moe_downcast_mxfp4", "moe_upcast_mxfp4", "moe_grouped_gemm", "moe_reduce", "moe_swiglu",
                     "moe_weight_layout_to_b200", "moe_weight_layout_from_b200", "moe_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from triton_b200 import _lib
    lib = _lib.load()
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_functions():
        assert hasattr(raw, name), f"libmoe_b200.so does not export {name}"
        assert name in _lib.PROTOTYPES, f"_lib.PROTOTYPES lacks {name}"
    assert lib.moe_abi_version() >= 1


def test_argument_errors_are_reported_not_raised_in_c():
    from triton_b200 import _lib
    lib = _lib.load()
    # quantised axis not a multiple of 32: rejected before any CUDA call
    st = lib.moe_downcast_mxfp4(None, _lib.MOE_BF16, 1, 1, 48, 0, 48, 1, None, None, 0, None)
    assert st == 1
    assert b"multiple of 32" in lib.moe_last_error()
    with pytest.raises(ValueError):
        _lib.check(st, "moe_downcast_mxfp4")
    # zero-sized problems succeed without touching the device
    assert lib.moe_downcast_mxfp4(None, _lib.MOE_BF16, 0, 4, 64, 0, 64, 1, None, None, 0, None) == 0
    assert lib.moe_topk_fwd(None, _lib.MOE_F32, 0, 8, 2, 1, 8, None, 2, None, 2, None, 1, 32, None, 0, None) == 0


def test_operators_refuse_cpu_tensors():
    import torch
    import triton_b200
    with pytest.raises(ValueError):
        triton_b200.downcast_to_mxfp(torch.zeros(4, 64, dtype=torch.bfloat16), torch.uint8, axis=-1)
