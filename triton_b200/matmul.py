"""Ragged grouped GEMM with gather / scatter and fused epilogue (triton_kernels/matmul.py:245-766):

    y[rows(e)] = act((x[gather(rows(e))] @ w[e] + bias[e] * betas) * out_alpha) * gammas

`matmul` keeps the reference's signature and argument meaning.  The body validates, allocates the
output through torch and makes one call into libmoe_b200 (`moe_grouped_gemm`), which picks the tcgen05
kernel for bf16 activations x MXFP4 weights in the B200 tiled layouts and the SIMT kernel otherwise."""
from dataclasses import dataclass
from enum import Enum, auto
from typing import Callable, Sequence

import torch

from . import _lib
from .matmul_details.opt_flags import (InapplicableConstraint, get_idle_sms, reset_opt_flags_constraints,  # noqa: F401
                                       resolve_kernel_choice, resolve_tile_m, resolve_tile_n,
                                       scoped_opt_flags_constraints, set_idle_sms,
                                       update_opt_flags_constraints)
from .numerics import InFlexData, OutFlexData
from .specialize import FnSpecs
from .tensor import FP4, RaggedTensorMetadata, Tensor, convert_layout, wrap_torch_tensor
from .tensor_details.layout import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout, B200MXScaleLayout,
                                    B200MXValueLayout, BlackwellMXScaleLayout, BlackwellMXValueLayout, StridedLayout)


@dataclass(frozen=True)
class FusedActivation:
    specs: FnSpecs = FnSpecs.default()
    fn_args: tuple = tuple()


@dataclass
class FusedComm:
    """Output rows stored straight into buffers of several devices (matmul.py:60-79 of the reference).

    out_handles: device addresses (ints) of one [rows_per_shard, N_out] buffer per shard, this rank's own included,
    peer-mapped memory for the others.  The reference takes a JIT closure `map_dst_coord`; the only map built here is
    the block map the expert-parallel combine needs: output row r (after scatter_indx) is row r % rows_per_shard of
    shard r // rows_per_shard.  `local` is this rank's buffer as a tensor: it carries dtype and row pitch and is
    what `matmul` returns."""
    out_handles: Sequence[int]
    rows_per_shard: int
    local: torch.Tensor
    map_dst_coord: object = "block_rows"
    reduce_rank: int = 0
    n_reduce_shards: int = 1


@dataclass(frozen=True)
class Epilogue:
    specs: FnSpecs = FnSpecs.default()
    fn_arg_values_matmul: tuple = tuple()
    fn_arg_values_finalize: tuple = tuple()
    effective_itemsize: float | None = None


class FnName(Enum):
    QUANTIZE_MXFP8 = auto()
    QUANTIZE_MXFP4 = auto()
    QUANTIZE_NVFP4 = auto()


@dataclass(frozen=True)
class FlexCtx:
    lhs_data: InFlexData = InFlexData()
    rhs_data: InFlexData = InFlexData()
    out_data: OutFlexData = OutFlexData()
    acc_data: InFlexData = InFlexData()


@dataclass
class PrecisionConfig:
    max_num_imprecise_acc: int | None = None
    allow_tf32: bool = True
    flex_ctx: FlexCtx = FlexCtx()
    acc_scale: float = 1.0
    flexpoint_saturate_inf: bool = False
    report_quantization_err_fn: Callable | None = None
    a_mx_scale: torch.Tensor | Tensor | None = None
    a_mx_tensor_scale: torch.Tensor | None = None
    a_microblock_size: int | None = None
    b_mx_scale: torch.Tensor | Tensor | None = None
    b_mx_tensor_scale: torch.Tensor | None = None
    b_microblock_size: int | None = None
    c_mx_scale: torch.Tensor | Tensor | None = None
    c_microblock_size: int | None = None
    c_value_pack_factor: int = 1
    out_dtype: torch.dtype | None = None
    intermediate_out_dtype: torch.dtype | None = None
    enforce_bitwise_invariance: bool = False


def matmul_set_idle_sms(num_idle_sms):
    set_idle_sms(num_idle_sms)


_status_words = {}
_scale_cache = {}


def _status_word(device):
    key = torch.device(device).index
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


_STATUS_TEXT = {
    101: "tcgen05 kernel: the MMA thread waited for a free accumulator", 102: "tcgen05 kernel: the MMA thread waited for activations",
    103: "tcgen05 kernel: the MMA thread waited for dequantised weights", 104: "tcgen05 kernel: the final MMA drain",
    201: "tcgen05 kernel: the weight producer waited for a free stage", 301: "tcgen05 kernel: the activation loader waited for a free stage",
    401: "tcgen05 kernel: the dequantiser waited for packed weights", 402: "tcgen05 kernel: the dequantiser waited for a free stage",
    501: "tcgen05 kernel: the epilogue waited for an accumulator",
    601: "block-scaled kernel: the producer waited for a free stage", 602: "block-scaled kernel: the MMA thread waited for a stage",
    603: "block-scaled kernel: the MMA thread waited for a free accumulator", 604: "block-scaled kernel: the epilogue waited for an accumulator",
    605: "block-scaled kernel: the final MMA drain", 606: "block-scaled kernel: the MMA thread waited for scales",
    607: "block-scaled kernel: a scale loader waited for a stage",
    801: "router kernel: the producer waited for a free stage", 802: "router kernel: the MMA thread waited for a stage",
    803: "router kernel: the final MMA drain", 804: "router kernel: the selection waited for the accumulator",
    901: "expert-parallel peer barrier: a rank did not arrive within the limit; the step after it read stale peer buffers",
}


def status_message(code: int) -> str:
    """Text for a device status code (the word every kernel with bounded waits writes when a wait expires)."""
    return _STATUS_TEXT.get(code, "a bounded wait expired inside a kernel")


def matmul_check_status(device=None):
    """Synchronise and raise if a bounded wait expired since the last check: a pipeline wait inside a tensor-core
    kernel (codes 1xx-8xx) or an expert-parallel peer barrier (901).  Expert-parallel callers should poll this once
    per step or batch: after a barrier time-out the step carries on with stale peer buffers and its result is wrong."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_word(dev)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"device status {code}: {status_message(code)}")


def _canonical_scale(b_scale: Tensor):
    """[E, K/32, N] view of an MX scale tensor stored in the reference's Blackwell scale layout (unswizzled
    once and remembered while the storage tensor is alive)."""
    data = b_scale.storage.data
    key = (data.data_ptr(), tuple(b_scale.shape))
    hit = _scale_cache.get(key)
    if hit is not None and hit[0]() is data:
        return hit[1]
    import weakref
    canon = b_scale.storage.layout.make_transformation(list(b_scale.shape), False).unswizzle_data(data).contiguous()
    _scale_cache[key] = (weakref.ref(data), canon)
    return canon


def matmul(a, b, bias,
           a_ragged_metadata: RaggedTensorMetadata | None = None,
           b_ragged_metadata: RaggedTensorMetadata | None = None,
           gather_indx: torch.Tensor | None = None,
           scatter_indx: torch.Tensor | None = None,
           precision_config: PrecisionConfig | None = None,
           betas: torch.Tensor | None = None,
           gammas: torch.Tensor | None = None,
           out_alpha: float | None = None,
           c: torch.Tensor | None = None,
           fused_comm=None,
           fused_activation: FusedActivation | None = None,
           epilogue: Epilogue | None = None,
           c_acc_in: torch.Tensor | None = None):
    """Y[idxs_y_m(e), :] = matmul(X[idxs_x_m(e), :], W[e, :, :]) for every expert e, with the epilogue above.

    a: [M, K] activations (bf16 / fp16 / fp32), K contiguous.  b: [E, K, N] (or [K, N]) dense tensor of the
    same dtype, or an FP4 `Tensor` / uint8 tensor packed along K together with
    `precision_config.b_mx_scale` ([E, K/32, N] e8m0).  a_ragged_metadata splits the (gathered) rows into
    one slice per expert.  gather_indx[m] is the row of `a` read for problem row m, scatter_indx[m] the row of
    the output written (-1 drops it); betas / gammas are per problem row, in expert-sorted order.
    """
    if a.ndim == 3:
        raise NotImplementedError("batched (3-D) activations are outside the MoE path")
    if b_ragged_metadata is not None:
        raise NotImplementedError("ragged-K (weight-gradient) matmul is outside the MoE path")
    if fused_comm is not None:
        if fused_comm.map_dst_coord != "block_rows" or fused_comm.n_reduce_shards != 1:
            raise NotImplementedError("fused_comm: only the block-of-rows destination map is implemented")
        if c is not None:
            raise ValueError("fused_comm writes into its own buffers: do not pass c")
        if len(fused_comm.out_handles) > _lib.MOE_MAX_PEERS:
            raise NotImplementedError(f"fused_comm: at most {_lib.MOE_MAX_PEERS} shards")
    if c_acc_in is not None:
        raise NotImplementedError("c_acc_in is not implemented")
    if precision_config is None:
        precision_config = PrecisionConfig()
    if fused_activation is None:
        fused_activation = FusedActivation(FnSpecs.default(), tuple())
    if epilogue is not None and epilogue.specs.name != "dflt":
        raise NotImplementedError("quantising epilogues are not implemented")
    pc = precision_config
    if pc.c_mx_scale is not None:
        raise NotImplementedError("microscaled outputs are not implemented")
    a_scale = pc.a_mx_scale
    if a_scale is not None:
        assert pc.a_microblock_size in (None, 32), "only 32-element e8m0 micro-blocks are supported"
        if isinstance(a_scale, Tensor):
            if not isinstance(a_scale.storage.layout, StridedLayout):
                raise NotImplementedError("a_mx_scale must be a plain [M, K/32] tensor")
            a_scale = a_scale.storage.data
    fc = pc.flex_ctx
    if any(s is not None for s in (fc.lhs_data.scale, fc.rhs_data.scale, fc.out_data.expected_scale, fc.acc_data.scale)):
        raise NotImplementedError("flexpoint scales are not implemented")
    kernel_choice = resolve_kernel_choice()
    if isinstance(a, Tensor):
        a = a.storage.data
    assert a.ndim == 2
    if a.stride(-1) != 1:
        a = a.contiguous()
    lib = _lib.load()
    dev = a.device
    args = _lib.MoeGemmArgs()
    keep = []                                           # temporaries that must outlive the launch call

    # ---- weights --------------------------------------------------------------------------------------
    b_scale = pc.b_mx_scale
    if b_scale is not None:
        assert pc.b_microblock_size in (None, 32), "only 32-element e8m0 micro-blocks are supported"
        if not isinstance(b, Tensor):
            assert b.dtype == torch.uint8, "MX weights must be packed e2m1 (uint8)"
            b = wrap_torch_tensor(b, dtype=FP4)
        if not isinstance(b_scale, Tensor):
            b_scale = wrap_torch_tensor(b_scale)
        assert b.dtype == FP4, "only MXFP4 weights are supported with b_mx_scale"
        shape = list(b.shape)
        if len(shape) == 2:
            shape = [1] + shape
        E, K, N = shape
        vl, sl = b.storage.layout, b_scale.storage.layout
        if (type(vl) in (B200MXValueLayout, B200BlockScaledValueLayout)) != \
                (type(sl) in (B200MXScaleLayout, B200BlockScaledScaleLayout)) or \
                isinstance(vl, B200BlockScaledValueLayout) != isinstance(sl, B200BlockScaledScaleLayout):
            raise ValueError("B200 tiled weights need values and scales in the matching pair of B200 layouts")
        if isinstance(vl, B200BlockScaledValueLayout):
            args.w_kind = _lib.MOE_W_MX4_B200MX
            args.w, args.w_scale = b.storage.data.data_ptr(), b_scale.storage.data.data_ptr()
        elif isinstance(vl, B200MXValueLayout):
            args.w_kind = _lib.MOE_W_MX4_B200
            args.w, args.w_scale = b.storage.data.data_ptr(), b_scale.storage.data.data_ptr()
        else:
            wd = b.storage.data
            if wd.ndim == 2:
                wd = wd.unsqueeze(0)
            if isinstance(vl, (StridedLayout, BlackwellMXValueLayout)):
                assert wd.stride(-2) == 1, "MXFP4 weights must be packed and contiguous along K"
            else:
                raise NotImplementedError(f"weight value layout {vl} is not supported")
            if isinstance(sl, StridedLayout):
                sd = b_scale.storage.data
                if sd.ndim == 2:
                    sd = sd.unsqueeze(0)
            elif isinstance(sl, BlackwellMXScaleLayout):
                sd = _canonical_scale(b_scale)
                if sd.ndim == 2:
                    sd = sd.unsqueeze(0)
            else:
                raise NotImplementedError(f"weight scale layout {sl} is not supported")
            assert tuple(sd.shape) == (E, K // 32, N), f"scale shape {tuple(sd.shape)} != {(E, K // 32, N)}"
            keep += [wd, sd]
            args.w_kind = _lib.MOE_W_MX4_CANONICAL
            args.w, args.w_scale = wd.data_ptr(), sd.data_ptr()
            args.w_stride_e, args.w_stride_k, args.w_stride_n = wd.stride(0), 1, wd.stride(2)
            args.ws_stride_e, args.ws_stride_k, args.ws_stride_n = sd.stride(0), sd.stride(1), sd.stride(2)
    else:
        if isinstance(b, Tensor):
            b = b.storage.data
        assert b.dtype == a.dtype, "dense weights must have the activation dtype"
        wd = b if b.ndim == 3 else b.unsqueeze(0)
        E, K, N = wd.shape
        keep.append(wd)
        args.w_kind = _lib.MOE_W_DENSE
        args.w = wd.data_ptr()
        args.w_stride_e, args.w_stride_k, args.w_stride_n = wd.stride(0), wd.stride(1), wd.stride(2)
    assert a.shape[-1] == K, f"inner dimensions differ: {a.shape[-1]} vs {K}"
    if a.dtype == torch.float8_e4m3fn or a_scale is not None:
        # e4m3 / MXFP8 activations exist on the block-scaled tensor-core path only
        if a.dtype != torch.float8_e4m3fn:
            raise NotImplementedError("a_mx_scale is implemented for e4m3 activations (MXFP8)")
        if args.w_kind != _lib.MOE_W_MX4_B200MX:
            raise NotImplementedError("e4m3 / MXFP8 activations need MXFP4 weights in B200BlockScaledValueLayout / "
                                      "B200BlockScaledScaleLayout")
        if pc.out_dtype is None:
            raise ValueError("e4m3 activations: set precision_config.out_dtype (bf16 or fp32)")
        if a_scale is not None:
            assert a_scale.dtype == torch.uint8 and tuple(a_scale.shape) == (a.shape[0], K // 32), \
                f"a_mx_scale must be uint8 [M, K/32], got {a_scale.dtype} {tuple(a_scale.shape)}"
            if a_scale.stride(-1) != 1:
                a_scale = a_scale.contiguous()
            keep.append(a_scale)
            args.x_scale, args.ld_x_scale = a_scale.data_ptr(), a_scale.stride(0)

    # ---- shapes / output ------------------------------------------------------------------------------
    M = a.shape[0] if gather_indx is None else gather_indx.shape[0]
    if scatter_indx is not None:
        assert scatter_indx.shape[0] == M, "scatter_indx must have one entry per problem row"
    red_n = fused_activation.specs.reduction_n
    act_name = fused_activation.specs.name
    if act_name not in ("dflt", "swiglu"):
        raise NotImplementedError(f"fused activation {act_name!r} is not implemented")
    assert (act_name == "swiglu") == (red_n == 2), "swiglu halves N (reduction_n == 2)"
    out_rows = M if scatter_indx is None else scatter_indx.shape[0]
    out_dtype = pc.out_dtype or a.dtype
    out_shape = (out_rows, N // red_n)
    if fused_comm is not None:
        c = fused_comm.local
        assert c.ndim == 2 and c.shape[1] == N // red_n and c.stride(-1) == 1 and c.dtype == out_dtype
        assert c.shape[0] == fused_comm.rows_per_shard
    elif c is None:
        c = torch.empty(out_shape, dtype=out_dtype, device=dev)
    else:
        if c.ndim == 3 and c.shape[0] == 1:
            c = c[0]
        assert tuple(c.shape) == out_shape and c.stride(-1) == 1 and c.dtype == out_dtype
    if M == 0 or N == 0:
        return c
    if a_ragged_metadata is None:
        assert E == 1, "several weight matrices need a_ragged_metadata"
    # A plain dense product (the router's logits = x @ Wg + bg, bench/bench_mlp.py:70 of the reference) is a library
    # GEMM: cuBLAS through torch, fp32 accumulation, with the epilogue terms that apply to it.
    if (args.w_kind == _lib.MOE_W_DENSE and kernel_choice == "auto" and a_ragged_metadata is None and gather_indx is None
            and scatter_indx is None and fused_comm is None and act_name == "dflt" and betas is None and gammas is None
            and a.dtype in (torch.bfloat16, torch.float16) and a.is_cuda):
        try:
            y = torch.mm(a, wd[0], out_dtype=torch.float32)      # fp32 out of the library GEMM: one rounding at the end
        except (TypeError, RuntimeError):
            y = torch.mm(a, wd[0]).float()
        if bias is not None:
            y = y + bias.reshape(1, -1).float()
        if out_alpha is not None:
            y = y * float(out_alpha)
        c.copy_(y)
        return c

    def i32(t):
        if t is None:
            return None
        t = t if t.dtype == torch.int32 else t.to(torch.int32)
        t = t if t.is_contiguous() else t.contiguous()
        keep.append(t)
        return t.data_ptr()

    def f32v(t):
        if t is None:
            return None
        t = t if t.dtype == torch.float32 else t.float()
        t = t if t.is_contiguous() else t.contiguous()
        keep.append(t)
        return t.data_ptr()

    args.x, args.x_dtype, args.ld_x, args.rows_x = a.data_ptr(), _lib.dtype_code(a.dtype), a.stride(0), a.shape[0]
    args.E, args.K, args.N, args.M = E, K, N, M
    if a_ragged_metadata is not None:
        md = a_ragged_metadata
        assert md.block_offs_data.stride(1) == 1 and md.block_schedule_data.stride(1) == 1
        args.slice_sizes, args.slice_offs = md.slice_sizes.data_ptr(), md.slice_offs.data_ptr()
        args.block_offs_16, args.block_sched_16 = md.block_offs_data.data_ptr(), md.block_schedule_data.data_ptr()
        args.ld_block_offs, args.ld_block_sched = md.block_offs_data.stride(0), md.block_schedule_data.stride(0)
    if bias is not None:
        if bias.ndim == 1:
            bias = bias.view(1, -1)
        assert bias.shape[-1] == N and bias.stride(-1) == 1
        args.bias, args.bias_dtype, args.ld_bias = bias.data_ptr(), _lib.dtype_code(bias.dtype), bias.stride(0)
    args.gather_indx, args.scatter_indx = i32(gather_indx), i32(scatter_indx)
    args.betas, args.gammas = f32v(betas), f32v(gammas)
    if out_alpha is not None:
        args.out_alpha, args.has_out_alpha = float(out_alpha), 1
    if act_name == "swiglu":
        alpha, limit = fused_activation.fn_args
        args.activation, args.act_alpha = _lib.MOE_ACT_SWIGLU, float(alpha)
        args.act_limit, args.act_has_limit = (float(limit), 1) if limit is not None else (0.0, 0)
    args.y, args.y_dtype, args.ld_y = c.data_ptr(), _lib.dtype_code(c.dtype), c.stride(0)
    if fused_comm is not None:
        args.n_y_peers, args.y_rows_per_peer = len(fused_comm.out_handles), int(fused_comm.rows_per_shard)
        for i, h in enumerate(fused_comm.out_handles):
            args.y_peers[i] = int(h)
    args.kernel = {"auto": _lib.MOE_GEMM_AUTO, "simt": _lib.MOE_GEMM_SIMT, "tcgen05": _lib.MOE_GEMM_TCGEN05,
                   "tcgen05-pair": _lib.MOE_GEMM_TCGEN05_PAIR, "stream": _lib.MOE_GEMM_STREAM,
                   "mx": _lib.MOE_GEMM_MX, "mx-f8": _lib.MOE_GEMM_MX_F8, "mx-f4": _lib.MOE_GEMM_MX_F4}[kernel_choice]
    args.tile_m, args.tile_n = resolve_tile_m(), resolve_tile_n()
    args.idle_sms = get_idle_sms()
    args.status = _status_word(dev).data_ptr()
    if args.w_kind == _lib.MOE_W_MX4_B200MX:
        ws_bytes = lib.moe_gemm_mx_workspace_bytes(args)
        ws = torch.empty(ws_bytes + 1024, dtype=torch.uint8, device=dev)        # token blocks in the MMA's operand layout
        keep.append(ws)
        args.mx_workspace = (ws.data_ptr() + 1023) // 1024 * 1024
        args.mx_workspace_bytes = ws_bytes
    if gather_indx is not None and args.w_kind == _lib.MOE_W_MX4_B200 and a.dtype == torch.bfloat16 and M >= 2048:
        scratch = torch.empty(M * K, dtype=torch.bfloat16, device=dev)   # the library decides whether to use it
        keep.append(scratch)
        args.gather_scratch, args.gather_scratch_bytes = scratch.data_ptr(), scratch.numel() * 2
    st = lib.moe_grouped_gemm(args, _lib.stream())
    if st == 3:
        raise InapplicableConstraint(lib.moe_last_error().decode(errors="replace"))
    _lib.check(st, "moe_grouped_gemm")
    return c


matmul_ogs = matmul          # the name this operator had in earlier releases of the reference
