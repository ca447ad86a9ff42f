"""User-visible tuning overrides for `matmul` (triton_kernels/matmul_details/opt_flags.py:482-532).

The constraint dictionary is context-local.  Keys understood here: ``kernel`` ("auto", "simt", "tcgen05-pair", "stream",
"tcgen05").  The reference's tile-shape keys (block_m, block_n, block_k, num_stages, split_k,
is_persistent, epilogue_subtile, ...) are accepted and ignored when they cannot matter, and raise
InapplicableConstraint when they ask for something the CUDA kernels do not implement (split_k > 1)."""
from contextlib import contextmanager
from contextvars import ContextVar

_opt_flags_constraints: ContextVar = ContextVar("opt_flags_constraints", default=None)
_idle_sms = 0

_IGNORED_KEYS = {"block_m", "block_n", "block_k", "num_stages", "is_persistent", "epilogue_subtile", "fused_scatter",
                 "idle_sms", "swap_xw", "disable_mx4_block_swap", "occupancy_target", "num_warps", "group_m", "clc"}


class InapplicableConstraint(Exception):
    pass


def set_idle_sms(num_idle_sms: int):
    """SMs the persistent grouped-GEMM kernels leave without a CTA, so that kernels on another stream (the
    expert-parallel row pulls) run beside them (triton_kernels/matmul.py:239-243)."""
    global _idle_sms
    _idle_sms = int(num_idle_sms)


def get_idle_sms() -> int:
    return _idle_sms


def get_opt_flags_constraints() -> dict:
    c = _opt_flags_constraints.get()
    return {} if c is None else c


def update_opt_flags_constraints(constraints: dict):
    updated = get_opt_flags_constraints().copy()
    updated.update(constraints)
    _opt_flags_constraints.set(updated)


def reset_opt_flags_constraints():
    _opt_flags_constraints.set(None)


@contextmanager
def scoped_opt_flags_constraints(constraints):
    updated = get_opt_flags_constraints().copy()
    updated.update(constraints)
    token = _opt_flags_constraints.set(updated)
    try:
        yield
    finally:
        _opt_flags_constraints.reset(token)


def resolve_tile_m() -> int:
    """`block_m` constraint -> token rows per tile (0 = heuristic).  The bf16 tensor-core kernel knows 128 and 256,
    the block-scaled kernel 16, 32, 64 and 128; each kernel ignores a value it does not have."""
    bm = get_opt_flags_constraints().get("block_m")
    return bm if bm in (16, 32, 64, 128, 256) else 0


def resolve_tile_n() -> int:
    """`block_n` constraint -> weight rows per tile (0 = heuristic): 128 / 256 for the bf16 tensor-core kernel,
    128 / 384 for the block-scaled kernel."""
    bn = get_opt_flags_constraints().get("block_n")
    return bn if bn in (128, 256, 384) else 0


def resolve_kernel_choice() -> str:
    c = get_opt_flags_constraints()
    for k, v in c.items():
        if k == "kernel":
            if v not in ("auto", "simt", "tcgen05", "tcgen05-pair", "stream", "mx"):
                raise InapplicableConstraint(f"unknown kernel {v!r}")
        elif k == "split_k":
            if v not in (None, 1):
                raise InapplicableConstraint("split_k > 1 is not implemented")
        elif k not in _IGNORED_KEYS:
            raise InapplicableConstraint(f"unsupported opt_flags constraint {k!r}")
    return c.get("kernel", "auto")
