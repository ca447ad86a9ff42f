"""ctypes binding of libmoe_b200.so (declarations mirror include/moe_b200.h).

The library is the only compute path of this package: if it cannot be loaded, every operator
raises.  There is no CPU or eager-PyTorch fallback.
"""
import ctypes as C
from pathlib import Path

import torch

import os

_HERE = Path(__file__).resolve().parent
# MOE_B200_LIB points at an alternative build of the library (e.g. an instrumented one)
LIB_PATH = Path(os.environ["MOE_B200_LIB"]) if os.environ.get("MOE_B200_LIB") else _HERE / "libmoe_b200.so"

MOE_F32, MOE_F16, MOE_BF16, MOE_F8E4M3 = 0, 1, 2, 3
MOE_ROUND_UP, MOE_ROUND_DOWN = 0, 1
MOE_ACT_NONE, MOE_ACT_SWIGLU = 0, 1
MOE_W_DENSE, MOE_W_MX4_CANONICAL, MOE_W_MX4_B200, MOE_W_MX4_B200MX = 0, 1, 2, 3
MOE_GEMM_AUTO, MOE_GEMM_SIMT, MOE_GEMM_TCGEN05, MOE_GEMM_TCGEN05_PAIR, MOE_GEMM_STREAM, MOE_GEMM_MX = 0, 1, 2, 3, 4, 5
MOE_GEMM_MX_F8, MOE_GEMM_MX_F4 = 6, 7
MOE_MAX_PEERS = 16

_DTYPE_CODE = {torch.float32: MOE_F32, torch.float16: MOE_F16, torch.bfloat16: MOE_BF16,
               torch.float8_e4m3fn: MOE_F8E4M3}

i64, i32, vp, sz, f32 = C.c_int64, C.c_int, C.c_void_p, C.c_size_t, C.c_float


class MoeDeviceInfo(C.Structure):
    _fields_ = [("sm_count", i32), ("cc_major", i32), ("cc_minor", i32), ("smem_per_block_optin", sz),
                ("l2_bytes", sz), ("total_mem", sz)]


class MoeGemmArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("x_dtype", i32), ("ld_x", i64), ("rows_x", i64),
        ("w_kind", i32), ("w", vp), ("w_stride_e", i64), ("w_stride_k", i64), ("w_stride_n", i64),
        ("w_scale", vp), ("ws_stride_e", i64), ("ws_stride_k", i64), ("ws_stride_n", i64),
        ("E", i32), ("K", i32), ("N", i32),
        ("slice_sizes", vp), ("slice_offs", vp), ("block_offs_16", vp), ("block_sched_16", vp),
        ("ld_block_offs", i64), ("ld_block_sched", i64), ("M", i64),
        ("bias", vp), ("bias_dtype", i32), ("ld_bias", i64),
        ("gather_indx", vp), ("scatter_indx", vp), ("betas", vp), ("gammas", vp),
        ("out_alpha", f32), ("has_out_alpha", i32),
        ("activation", i32), ("act_alpha", f32), ("act_limit", f32), ("act_has_limit", i32),
        ("y", vp), ("y_dtype", i32), ("ld_y", i64),
        ("kernel", i32), ("tile_m", i32), ("tile_n", i32), ("status", vp),
        ("y_peers", vp * 16), ("n_y_peers", i32), ("y_rows_per_peer", i64),
        ("gather_scratch", vp), ("gather_scratch_bytes", i64),
        ("x_scale", vp), ("ld_x_scale", i64), ("mx_workspace", vp), ("mx_workspace_bytes", i64), ("idle_sms", i32),
    ]


# name -> (restype, argtypes); must list every symbol declared in include/moe_b200.h
PROTOTYPES = {
    "moe_last_error": (C.c_char_p, []),
    "moe_abi_version": (i32, []),
    "moe_launch_count": (C.c_uint64, []),
    "moe_device_info": (i32, [i32, C.POINTER(MoeDeviceInfo)]),
    "moe_downcast_mxfp4": (i32, [vp, i32, i64, i64, i64, i64, i64, i64, vp, vp, i32, vp]),
    "moe_upcast_mxfp4": (i32, [vp, vp, vp, i32, i64, i64, i64, i64, i64, i64, vp]),
    "moe_topk_fwd": (i32, [vp, i32, i64, i32, i32, i32, i64, vp, i64, vp, i64, vp, i64, i64, vp, i32, vp]),
    "moe_bitmatrix_metadata_workspace": (sz, [i64, i32, i32]),
    "moe_bitmatrix_metadata": (i32, [vp, i64, i64, i32, i32, vp, vp, vp, vp, vp, sz, vp]),
    "moe_route_workspace": (sz, [i64, i32, i32]),
    "moe_route": (i32, [vp, i32, i64, i32, i32, i32, i64, vp, i64, vp, i64, vp, i64, i64, vp, vp, vp, vp, vp, i64, vp, i64,
                        i64, vp, sz, vp]),
    "moe_router_topk_workspace_bytes": (sz, [i64, i64, i32]),
    "moe_router_topk": (i32, [vp, i64, i64, i64, vp, i64, vp, i32, i32, i32, i32, i32, vp, i64, vp, i32, i64, vp, i64, vp, i64,
                              i64, vp, sz, vp, vp]),
    "moe_bitmatrix_metadata_noalloc_capacity": (sz, []),
    "moe_bitmatrix_metadata_noalloc": (i32, [vp, i64, i64, i32, i32, vp, vp, vp, vp, vp]),
    "moe_ragged_metadata": (i32, [vp, i32, vp, vp, i64, vp, i64, i64, vp]),
    "moe_ragged_metadata_remap": (i32, [vp, vp, vp, i64, vp, i64, i64, vp, i32, vp, vp, vp, vp, vp]),
    "moe_swiglu": (i32, [vp, i64, vp, i64, i32, i64, i64, f32, f32, i32, vp, vp]),
    "moe_reduce": (i32, [vp, i32, i64, i64, i64, i64, i64, i64, vp, i32, i64, i64, i64, vp, i64, i64, i64, vp, i32,
                         i64, i64, vp]),
    "moe_weight_b200_value_bytes": (sz, [i32, i32, i32]),
    "moe_weight_b200_scale_bytes": (sz, [i32, i32, i32]),
    "moe_weight_layout_to_b200": (i32, [vp, i64, i64, vp, i64, i64, i64, i32, i32, i32, vp, vp, vp]),
    "moe_weight_layout_from_b200": (i32, [vp, vp, i32, i32, i32, vp, vp, vp]),
    "moe_weight_layout_to_b200mx": (i32, [vp, i64, i64, vp, i64, i64, i64, i32, i32, i32, vp, vp, vp]),
    "moe_weight_layout_from_b200mx": (i32, [vp, vp, i32, i32, i32, vp, vp, vp]),
    "moe_grouped_gemm": (i32, [C.POINTER(MoeGemmArgs), vp]),
    "moe_gemm_mx_workspace_bytes": (sz, [C.POINTER(MoeGemmArgs)]),
    "moe_tensor_roof": (i32, [i32, i32, C.POINTER(C.c_double), vp, vp]),
    "moe_ep_keys": (i32, [vp, vp, vp, i64, i32, i32, vp, vp]),
    "moe_ep_pull_index": (i32, [vp, vp, vp, vp, i64, i32, vp, vp, vp]),
    "moe_ep_combine_index": (i32, [vp, vp, vp, i64, i64, i64, vp, vp]),
    "moe_gather_rows": (i32, [vp, i64, vp, i64, i64, vp, i64, vp]),
    "moe_gather_rows_peers": (i32, [vp, i32, i64, i64, vp, i64, i64, vp, i64, vp]),
    "moe_peer_barrier": (i32, [vp, i32, i32, vp, vp, vp]),
    "moe_allgather_peers": (i32, [vp, i32, i64, vp, vp]),
    "moe_gather_reduce_rows_peers": (i32, [vp, i32, i64, i64, vp, i64, i32, i64, vp, i64, vp]),
    "moe_gather_reduce_rows": (i32, [vp, i64, vp, i64, i32, i64, vp, i64, vp]),
    "moe_scatter_rows": (i32, [vp, i64, vp, i64, i64, vp, i64, vp]),
}

_lib = None


class MoeLibraryError(RuntimeError):
    pass


def load():
    """Load libmoe_b200.so once.  Raises MoeLibraryError if it is missing (build it with
    ``python -m triton_b200.build``); nothing in this package works without it."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise MoeLibraryError(f"{LIB_PATH} not found: build it with `python -m triton_b200.build` "
                              "(this package has no fallback path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise MoeLibraryError(f"{LIB_PATH} does not export {name}") from e
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(status: int, what: str = ""):
    if status != 0:
        msg = load().moe_last_error().decode(errors="replace")
        exc = NotImplementedError if status == 3 else (ValueError if status == 1 else RuntimeError)
        raise exc(f"{what or 'libmoe_b200'} failed (status {status}): {msg}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}") from None


def ptr(t):
    """Device pointer of a tensor (None -> NULL).  The tensor must live on a CUDA device."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("triton_b200 operators take CUDA tensors only (no CPU path)")
    return t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


_zero_scratch = {}
ZERO_SCRATCH_CAP = 160 << 20


def zero_scratch(device, nbytes):
    """A device buffer that is all zero between calls, for the kernels that keep partial sums of K slices in global
    memory (they want it zero and leave it zero).  One buffer per device, cleared when it is allocated and grown on demand
    up to ZERO_SCRATCH_CAP; calls that use it must not overlap on the GPU (one stream, or the caller's own ordering).
    -> tensor, or None when there is none of that size and one cannot be made now: during CUDA-graph capture (the buffer
    would belong to the graph), or above the cap.  Callers then take their form without K slices."""
    import torch
    dev = torch.device(device)
    t = _zero_scratch.get(dev.index)
    if t is not None and t.numel() >= nbytes:
        return t
    if nbytes > ZERO_SCRATCH_CAP or torch.cuda.is_current_stream_capturing():
        return None
    grow = max(int(nbytes), 32 << 20)
    t = torch.zeros(grow, dtype=torch.uint8, device=dev)
    _zero_scratch[dev.index] = t
    return t
