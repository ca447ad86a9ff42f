"""User-visible tuning overrides for `matmul` (triton_kernels/matmul_details/opt_flags.py:482-532).

The constraint dictionary is context-local.  Keys understood here: ``kernel`` ("auto", "simt", "tcgen05", "tcgen05-pair",
"stream", "mx", "mx-f8", "mx-f4"), ``block_m`` (token rows per tile: 16 / 32 / 64 / 128 for the block-scaled kernel, 128 / 256 for the bf16
tensor-core kernel, whose 128-row tile spans only the rows present in steps of 16), ``block_n`` (128 / 256 / 384),
``idle_sms``.  Every other tile-shape key of the reference may be given only the value the CUDA kernels are built with
(``block_k`` 64 or 128, ``split_k`` 1, ``is_persistent`` True, the rest None); anything else raises
InapplicableConstraint, which the reference's tests treat as "skip"."""
from contextlib import contextmanager
from contextvars import ContextVar

_opt_flags_constraints: ContextVar = ContextVar("opt_flags_constraints", default=None)
_idle_sms = 0

# key -> values that the kernels can honour (None = "not constrained" is always accepted)
_APPLICABLE = {
    "block_m": {16, 32, 64, 128, 256}, "block_n": {128, 256, 384}, "block_k": {64, 128}, "split_k": {1},
    "is_persistent": {True},
    # fixed by the kernels: only "unconstrained" can be honoured
    "num_stages": set(), "epilogue_subtile": set(), "fused_scatter": set(), "swap_xw": set(), "disable_mx4_block_swap": set(),
    "occupancy_target": set(), "num_warps": set(), "group_m": set(), "clc": set(),
}


class InapplicableConstraint(Exception):
    pass


def set_idle_sms(num_idle_sms: int):
    """SMs the persistent grouped-GEMM kernels leave without a CTA, so that kernels on another stream (the
    expert-parallel row pulls) run beside them (triton_kernels/matmul.py:239-243)."""
    global _idle_sms
    _idle_sms = int(num_idle_sms)


def get_idle_sms() -> int:
    v = get_opt_flags_constraints().get("idle_sms")
    return _idle_sms if v is None else int(v)


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
            if v not in ("auto", "simt", "tcgen05", "tcgen05-pair", "stream", "mx", "mx-f8", "mx-f4"):
                raise InapplicableConstraint(f"unknown kernel {v!r}")
        elif k == "idle_sms":
            if v is not None and (not isinstance(v, int) or v < 0):
                raise InapplicableConstraint(f"idle_sms must be a non-negative integer, got {v!r}")
        elif k in _APPLICABLE:
            if v is not None and v not in _APPLICABLE[k]:
                allowed = sorted(_APPLICABLE[k], key=str) or ["unconstrained"]
                raise InapplicableConstraint(f"opt_flags constraint {k}={v!r} cannot be honoured (possible: {allowed})")
        else:
            raise InapplicableConstraint(f"unsupported opt_flags constraint {k!r}")
    return c.get("kernel", "auto")
