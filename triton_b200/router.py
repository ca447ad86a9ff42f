"""Router product fused with the top-k selection: `topk(matmul(x, wg, bg), k)` in one kernel.

The reference computes the router logits with its general `matmul` and hands them to `topk`
(triton_kernels bench/bench_mlp.py:70, topk.py:106-141); here the logits stay in tensor memory and the selection,
the softmax over the selected logits and the expert bitmatrix happen in the GEMM's epilogue (`moe_router_topk`)."""
import torch

from . import _lib
from .matmul import _status_word
from .tensor import BIT, SparseMatrix, wrap_torch_tensor
from .topk import topk


def prepare_router_weight(wg: torch.Tensor) -> torch.Tensor:
    """-> Wg as the kernel reads it: logical shape [K, E] kept, memory [E, K] with K contiguous (stride(0) == 1).
    A weight that already has that memory order is returned as it is; do this once per layer, not per step."""
    assert wg.ndim == 2
    if wg.stride(0) == 1 and wg.stride(1) % 8 == 0 and wg.dtype == torch.bfloat16:
        return wg
    return wg.to(torch.bfloat16).t().contiguous().t()


def router_topk_supported(x, wg, k) -> bool:
    return (isinstance(x, torch.Tensor) and x.is_cuda and x.ndim == 2 and x.dtype == torch.bfloat16 and wg.dtype == torch.bfloat16
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0 and wg.stride(0) == 1 and wg.stride(1) % 8 == 0
            and wg.shape[1] <= 256 and k in (1, 2, 4, 8, 16) and k <= wg.shape[1] and x.data_ptr() % 16 == 0
            and wg.data_ptr() % 16 == 0)


def _two_steps(logits, k, apply_softmax, return_logits):
    sp = topk(logits, k, apply_softmax=apply_softmax)
    return (sp, logits.float()) if return_logits else sp


def router_topk(x: torch.Tensor, wg: torch.Tensor, bg, k: int, apply_softmax: bool = True, logits_dtype=None,
                return_logits: bool = False):
    """SparseMatrix of `topk(x @ wg + bg, k, apply_softmax)` (and the fp32 logits when `return_logits`).

    x [T, K] bf16; wg [K, E] bf16 -- in the memory order of `prepare_router_weight`, else it is re-laid-out on every
    call; bg [E] or None.  `logits_dtype` is the dtype the two-step form would give the logits (default x.dtype: bf16,
    i.e. every logit is rounded to bf16 before the selection, as `matmul` rounds its output); the routing weights come
    back in that dtype like `topk`'s.  Shapes the kernel does not take (more than 256 experts, k not a power of two up
    to 16, unaligned rows) run the two steps apart."""
    logits_dtype = x.dtype if logits_dtype is None else logits_dtype
    assert logits_dtype in (torch.bfloat16, torch.float32)
    wg = prepare_router_weight(wg)
    if not router_topk_supported(x, wg, k):
        logits = (x.float() @ wg.float() + (0 if bg is None else bg.float())).to(logits_dtype)
        return _two_steps(logits, k, apply_softmax, return_logits)
    lib = _lib.load()
    T, K = x.shape
    E = wg.shape[1]
    dev = x.device
    vals = torch.empty((T, k), dtype=logits_dtype, device=dev)
    indx = torch.empty((T, k), dtype=torch.int16, device=dev)
    words, t_pad = (E + 31) // 32, (T + 31) // 32 * 32
    bm_store = torch.empty((words, t_pad), dtype=torch.int32, device=dev)
    bm = bm_store.transpose(0, 1)[:T]
    logits = torch.empty((T, E), dtype=torch.float32, device=dev) if return_logits else None
    ws_bytes = lib.moe_router_topk_workspace_bytes(T, K, E)
    ws = _lib.zero_scratch(dev, ws_bytes) if ws_bytes > 0 else None
    if ws_bytes > 0 and ws is None:
        # no zeroed scratch to be had now (first use inside a graph capture): the two steps apart
        logits = torch.addmm(bg.to(x.dtype), x, wg) if bg is not None else x @ wg
        return _two_steps(logits.to(logits_dtype), k, apply_softmax, return_logits)
    if bg is not None and bg.dtype not in (torch.float32, torch.bfloat16):
        bg = bg.float()
    if T > 0:
        _lib.check(lib.moe_router_topk(_lib.ptr(x), T, K, x.stride(0), _lib.ptr(wg), wg.stride(1), _lib.ptr(bg),
                                       _lib.dtype_code(bg.dtype) if bg is not None else 0, E, k, int(bool(apply_softmax)),
                                       int(logits_dtype == torch.bfloat16), _lib.ptr(logits), E, _lib.ptr(vals),
                                       _lib.dtype_code(vals.dtype), vals.stride(0), _lib.ptr(indx), indx.stride(0), _lib.ptr(bm),
                                       bm.stride(0), bm.stride(1), _lib.ptr(ws), ws_bytes if ws is not None else 0,
                                       _status_word(dev).data_ptr(),
                                       _lib.stream()), "moe_router_topk")
    bitmatrix = wrap_torch_tensor(bm, dtype=BIT, shape=[T, E], shape_max=[T, None])
    sp = SparseMatrix(indx=indx, vals=vals, mask=bitmatrix)
    return (sp, logits) if return_logits else sp
