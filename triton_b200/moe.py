"""The MoE layer as the reference composes it from its operators
(python/triton_kernels/tests/test_distributed.py:213-247, bench/bench_mlp.py:60-96):

    routing -> [dispatch] -> fc1 (+bias, SwiGLU fused) -> fc2 (+bias, x routing weight) -> [combine exchange]
            -> k-way reduce

`MoeLayerWeights` holds MXFP4 expert weights already in the B200 tiled layouts."""
import ctypes
from dataclasses import dataclass

import torch

from .matmul import FusedActivation, PrecisionConfig, matmul
from .numerics_details.mxfp import downcast_to_mxfp
from .reduce import reduce
from .routing import route, routing  # noqa: F401
from .specialize import FnSpecs
from .swiglu import swiglu_fn
from .tensor import (FP4, Tensor, convert_layout, make_ragged_tensor_metadata, remap_ragged_tensor_metadata,
                     wrap_torch_tensor)
from .tensor_details.layout import make_default_matmul_mxfp4_w_layout, make_default_matmul_mxfp4_w_scale_layout
from .topk import topk


@dataclass
class MoeLayerWeights:
    w1: Tensor                 # FP4 [E, d_model, 2 * d_ff] (gate / linear columns interleaved)
    w1_scale: Tensor
    b1: torch.Tensor           # [E, 2 * d_ff]
    w2: Tensor                 # FP4 [E, d_ff, d_model]
    w2_scale: Tensor
    b2: torch.Tensor           # [E, d_model]
    alpha: float = 1.702
    limit: float | None = 7.0
    # canonical copies (packed along K), kept only when asked for (tests)
    w1_q: torch.Tensor | None = None
    w1_s: torch.Tensor | None = None
    w2_q: torch.Tensor | None = None
    w2_s: torch.Tensor | None = None
    # the same weights in the layouts of the block-scaled kernel (B200BlockScaledValueLayout / ...ScaleLayout); when
    # present, steps with few rows per expert run on it (see `use_block_scaled`)
    w1_bs: Tensor | None = None
    w1_bs_scale: Tensor | None = None
    w2_bs: Tensor | None = None
    w2_bs_scale: Tensor | None = None
    block_scaled_max_rows_per_expert: int = 48       # measured crossover: 32 rows per expert 1.3-1.45 x faster on the
                                                      # block-scaled kernel, 64 rows per expert 1.1 x slower

    @property
    def n_expts(self):
        return self.b1.shape[0]

    def use_block_scaled(self, n_rows: int) -> bool:
        """Few rows per expert (decode): the block-scaled kernel streams the packed weights straight into the MMA and
        is bound by HBM; with many rows per expert the bf16 kernel's larger token tiles win."""
        return self.w1_bs is not None and n_rows <= self.block_scaled_max_rows_per_expert * self.n_expts

    def fc_weights(self, n_rows: int):
        if self.use_block_scaled(n_rows):
            return self.w1_bs, self.w1_bs_scale, self.w2_bs, self.w2_bs_scale
        return self.w1, self.w1_scale, self.w2, self.w2_scale

    def weight_bytes(self):
        return sum(t.storage.data.numel() for t in (self.w1, self.w1_scale, self.w2, self.w2_scale)) + \
            self.b1.numel() * self.b1.element_size() + self.b2.numel() * self.b2.element_size()


def quantize_expert_weights(w: torch.Tensor):
    """bf16 [E, K, N] -> (FP4 values, e8m0 scales) quantised along K, in the default B200 layouts, plus the
    canonical tensors they were made from."""
    q, s = downcast_to_mxfp(w, torch.uint8, axis=1)
    tq = convert_layout(wrap_torch_tensor(q, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=-2))
    ts = convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=-2))
    return tq, ts, q, s


class _NoTimer:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _span(timer):
    """`timer` (optional) is a context-manager factory: timer() brackets each grouped-GEMM launch."""
    return timer() if timer is not None else _NoTimer()


def _activation(lw):
    return FusedActivation(FnSpecs("swiglu", swiglu_fn, ("alpha", "limit"), reduction_n=2), (lw.alpha, lw.limit))


def moe_layer_forward(x, logits, lw: MoeLayerWeights, k: int, gemm_timer=None):
    """x [T, d_model] bf16, logits [T, E] -> [T, d_model]: sum over the k selected experts of
    softmax-weight * (SwiGLU(x W1 + b1) W2 + b2).

    e4m3 activations (`x.dtype == torch.float8_e4m3fn`, the reference's fp8 mode: bench/bench_mlp.py `x_dtype="fp8"`) run
    both GEMMs on the block-scaled kernel at every size: fc1 writes e4m3 rows, fc2 reads them and writes bf16."""
    T = x.shape[0]
    ragged, sparse = route(logits, k, apply_softmax=True)
    md = sparse.mask_metadata
    n = T * k
    scatter_idx = md.col_sorted_indx                                    # sorted position -> flat (token, slot) row
    # token row and routing weight of every expert-sorted position, by one kernel (padding positions read no row)
    from . import _lib
    gather_idx = torch.empty(n, dtype=torch.int32, device=x.device)
    gammas = torch.empty(n, dtype=torch.float32, device=x.device)
    indx16 = sparse.indx if sparse.indx.dtype == torch.int16 else sparse.indx.to(torch.int16)
    _lib.check(_lib.load().moe_ep_pull_index(_lib.ptr(scatter_idx.reshape(-1)), _lib.ptr(indx16.contiguous()),
                                             _lib.ptr(sparse.vals.contiguous()), _lib.ptr(_all_local(logits.shape[1], x.device)),
                                             n, k, _lib.ptr(gather_idx), _lib.ptr(gammas), _lib.stream()), "moe_ep_pull_index")
    if x.dtype == torch.float8_e4m3fn:
        assert lw.w1_bs is not None, "e4m3 activations need the block-scaled copy of the weights"
        w1, w1_scale, w2, w2_scale = lw.w1_bs, lw.w1_bs_scale, lw.w2_bs, lw.w2_bs_scale
        pc1 = PrecisionConfig(b_mx_scale=w1_scale, b_microblock_size=32, out_dtype=torch.float8_e4m3fn)
        pc2 = PrecisionConfig(b_mx_scale=w2_scale, b_microblock_size=32, out_dtype=torch.bfloat16)
    else:
        w1, w1_scale, w2, w2_scale = lw.fc_weights(T * k)
        pc1 = PrecisionConfig(b_mx_scale=w1_scale, b_microblock_size=32)
        pc2 = PrecisionConfig(b_mx_scale=w2_scale, b_microblock_size=32)
    with _span(gemm_timer):
        h = matmul(x, w1, lw.b1, ragged, gather_indx=gather_idx, precision_config=pc1,
                   fused_activation=_activation(lw))
    with _span(gemm_timer):
        y = matmul(h, w2, lw.b2, ragged, scatter_indx=scatter_idx, precision_config=pc2, gammas=gammas)
    z, _ = reduce(y.view(T, k, -1), dim=1)
    return z


_all_local_cache = {}


def _all_local(n_expts, device):
    """int32 zeros [n_expts]: the "every expert lives here" table of moe_ep_pull_index."""
    key = (n_expts, torch.device(device).index)
    if key not in _all_local_cache:
        _all_local_cache[key] = torch.zeros(n_expts, dtype=torch.int32, device=device)
    return _all_local_cache[key]


class GraphedMoeLayer:
    """A layer forward for a fixed token count, captured once in a CUDA graph and replayed: at decode sizes the dozen
    launches of a step cost more host time than they run on the GPU, and in the expert-parallel layer the routing
    phase before the first GEMM is a chain of short launches.  `forward(x, logits) -> z` defaults to the single-GPU
    layer on `lw`; any forward without host synchronisation and without collectives can be passed instead (a capture
    of the expert-parallel step, whose NCCL barriers and all-gathers sit inside the graph, stopped making progress
    on 2 GPUs and is not used).  `__call__` copies the inputs into the graph's static buffers and returns a copy of the
    graph's static output tensor."""

    def __init__(self, lw: MoeLayerWeights, k: int, n_tokens: int, d_model: int, n_expts: int, device, warmup: int = 3,
                 forward=None):
        self.forward = forward if forward is not None else (lambda x, logits: moe_layer_forward(x, logits, lw, k))
        self.x = torch.zeros((n_tokens, d_model), dtype=torch.bfloat16, device=device)
        self.logits = torch.zeros((n_tokens, n_expts), dtype=torch.float32, device=device)
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):                  # lazy initialisation (kernel attributes, caches) happens here
            for _ in range(warmup):
                self.forward(self.x, self.logits)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.z = self.forward(self.x, self.logits)

    def replay(self):
        """Replay on the graph's own input buffers (`self.x`, `self.logits`); the result is `self.z`."""
        self.graph.replay()
        return self.z

    def __call__(self, x, logits):
        self.x.copy_(x, non_blocking=True)
        self.logits.copy_(logits, non_blocking=True)
        self.graph.replay()
        # a copy, so that the caller may still be reading one result (a download, say) while the next step replays
        return self.z.clone()


class HostStreamingLayer:
    """Layer steps fed from pinned host buffers and returning into pinned host buffers, pipelined over three streams:
    while step i computes, the inputs of step i + 1 are uploading and the result of step i - 1 is downloading (two
    device input slots).  `forward(x_dev, logits_dev) -> z_dev` is the layer (any of the forward functions above,
    bound to its weights).  Every `submit` copies that step's inputs in and its result out; `drain` waits for all of
    them."""

    def __init__(self, forward, n_tokens, d_model, n_expts, device, static_output=False):
        # static_output: `forward` returns the same tensor every call (a replayed CUDA graph): the next step then
        # waits until the previous result has left the device
        self.forward = forward
        self.static_output = static_output
        self.ev_out = torch.cuda.Event()
        self.dev = torch.device(device)
        self.s_in, self.s_out = torch.cuda.Stream(device=self.dev), torch.cuda.Stream(device=self.dev)
        self.x = [torch.empty((n_tokens, d_model), dtype=torch.bfloat16, device=self.dev) for _ in range(2)]
        self.logits = [torch.empty((n_tokens, n_expts), dtype=torch.float32, device=self.dev) for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_done = [torch.cuda.Event() for _ in range(2)]
        self.n = 0

    def submit(self, x_host, logits_host, z_host):
        b = self.n & 1
        main = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self.s_in):
            if self.n >= 2:
                self.s_in.wait_event(self.ev_done[b])          # the step that last read this slot has finished
            else:
                self.s_in.wait_stream(main)
            self.x[b].copy_(x_host, non_blocking=True)
            self.logits[b].copy_(logits_host, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        main.wait_event(self.ev_in[b])
        if self.static_output and self.n > 0:
            main.wait_event(self.ev_out)
        z = self.forward(self.x[b], self.logits[b])
        self.ev_done[b].record(main)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_done[b])
            z_host.copy_(z, non_blocking=True)
            z.record_stream(self.s_out)
            self.ev_out.record(self.s_out)
        self.n += 1

    def drain(self):
        torch.cuda.current_stream(self.dev).wait_stream(self.s_out)
        torch.cuda.current_stream(self.dev).wait_stream(self.s_in)


def _forward_ep_peer(x_local, sparse, lw_local, k, expt_assignment, pool, gemm_timer, mark=None, tokens_published=False):
    """Expert-parallel layer over peer-mapped buffers: the dispatch is one gather kernel that pulls every routed token
    row from its home rank's buffer into expert-sorted order (the layout fc1's TMA loads want); fc2 writes its rows
    into this rank's symmetric output buffer, and the combine is one kernel in which every token reads its k rows from
    the owners' buffers and sums them.  Both transfers are row-wise (512-byte warp accesses over NVLink; stores of
    16 bytes from the GEMM epilogue into peer memory ran at a seventh of that) and stream-ordered barriers replace the
    two all-to-alls: one before the dispatch (shared with the all-gather of the routing outputs when the caller put the
    tokens into the pool's buffer ahead of it: `tokens_published`) and one before the combine."""
    from . import _lib
    lib = _lib.load()
    mesh = pool.mesh
    W, rank = mesh.world_size, mesh.local_rank
    T_local, d = x_local.shape
    md = sparse.mask_metadata
    n = md.row_sorted_indx.shape[0]
    dev = x_local.device
    meta_global = make_ragged_tensor_metadata(md.col_sum, n)
    meta_local = remap_ragged_tensor_metadata(meta_global, expt_assignment.expt_map[rank, :])
    col = md.col_sorted_indx.reshape(-1)                               # flat (token * k + slot) of every position
    # positions whose expert lives here pull their token's row; all others are skipped (and never read by the GEMMs)
    src_row = torch.empty(n, dtype=torch.int32, device=dev)
    gammas = torch.empty(n, dtype=torch.float32, device=dev)
    mark = mark or (lambda name: None)
    indx16 = sparse.indx if sparse.indx.dtype == torch.int16 else sparse.indx.to(torch.int16)
    indx16 = indx16.contiguous()
    local_expt, owner = _ep_tables(expt_assignment, rank)
    mark("metadata")
    _lib.check(lib.moe_ep_pull_index(_lib.ptr(col), _lib.ptr(indx16), _lib.ptr(sparse.vals.contiguous()),
                                     _lib.ptr(local_expt), n, k, _lib.ptr(src_row), _lib.ptr(gammas), _lib.stream()),
               "moe_ep_pull_index")
    chunks = int(getattr(pool, "overlap_chunks", 1))
    w1, w1_scale, w2, w2_scale = lw_local.fc_weights(n // W)            # rows this rank multiplies, on average
    E_loc = lw_local.n_expts
    if lw_local.use_block_scaled(n // W) or E_loc < 2:
        chunks = 1
    chunks = max(1, min(chunks, E_loc))
    plan = None
    if chunks > 1:
        # Pipeline: the experts of this rank in `chunks` groups; the rows of group c + 1 are pulled on a side stream while
        # fc1 runs on group c.  Everything a group needs -- its pull index (rows of other groups: -2 = leave alone) and its
        # ragged metadata (other experts masked out, offsets kept global) -- is computed before the token barrier.
        bounds = [(E_loc * c) // chunks for c in range(chunks + 1)]
        plan = []
        for c in range(chunks):
            lo_e, hi_e = bounds[c], bounds[c + 1]
            table = torch.where((local_expt >= lo_e) & (local_expt < hi_e), local_expt - lo_e, torch.full_like(local_expt, -1))
            rows_c = torch.empty(n, dtype=torch.int32, device=dev)
            _lib.check(lib.moe_ep_pull_index(_lib.ptr(col), _lib.ptr(indx16), _lib.ptr(sparse.vals.contiguous()),
                                             _lib.ptr(table), n, k, _lib.ptr(rows_c), _lib.ptr(gammas), _lib.stream()),
                       "moe_ep_pull_index")
            plan.append((rows_c, remap_ragged_tensor_metadata(meta_global, table), lo_e, hi_e))
    if not tokens_published:                                           # (the caller did both ahead of the routing barrier)
        if x_local.data_ptr() != pool.xbuf.data_ptr():                 # a caller may keep its tokens in the pool's buffer
            pool.xbuf.copy_(x_local)
        pool.barrier()                                                 # every rank's tokens are in its buffer
    mark("pull index + token barrier")
    x_sorted = torch.empty((n, d), dtype=x_local.dtype, device=dev)
    ptrs = (ctypes.c_void_p * W)(*pool.x_ptrs)
    row_bytes = d * x_local.element_size()
    pc1 = PrecisionConfig(b_mx_scale=w1_scale, b_microblock_size=32)
    pc2 = PrecisionConfig(b_mx_scale=w2_scale, b_microblock_size=32)
    if plan is None:
        _lib.check(lib.moe_gather_rows_peers(ptrs, W, T_local, row_bytes, _lib.ptr(src_row), n, row_bytes, _lib.ptr(x_sorted),
                                             row_bytes, _lib.stream()), "moe_gather_rows_peers")
        mark("dispatch pull")
        with _span(gemm_timer):
            h = matmul(x_sorted, w1, lw_local.b1, a_ragged_metadata=meta_local, precision_config=pc1,
                       fused_activation=_activation(lw_local))
    else:
        from .matmul_details import opt_flags
        main = torch.cuda.current_stream(dev)
        side = pool.side_stream(dev)
        start = torch.cuda.Event()
        start.record(main)
        side.wait_event(start)
        pulled = []
        with torch.cuda.stream(side):
            for rows_c, _, _, _ in plan:
                _lib.check(lib.moe_gather_rows_peers(ptrs, W, T_local, row_bytes, _lib.ptr(rows_c), n, row_bytes,
                                                     _lib.ptr(x_sorted), row_bytes, side.cuda_stream), "moe_gather_rows_peers")
                ev = torch.cuda.Event()
                ev.record(side)
                pulled.append(ev)
        h = torch.empty((n, w1.shape[-1] // 2), dtype=x_local.dtype, device=dev)
        idle = int(getattr(pool, "overlap_idle_sms", 0))
        with _span(gemm_timer):
            for (rows_c, meta_c, lo_e, hi_e), ev in zip(plan, pulled):
                main.wait_event(ev)
                last = hi_e == E_loc
                with opt_flags.scoped_opt_flags_constraints({"idle_sms": None if last else idle}):
                    matmul(x_sorted, _expert_range(w1, lo_e, hi_e), lw_local.b1[lo_e:hi_e], a_ragged_metadata=meta_c,
                           precision_config=PrecisionConfig(b_mx_scale=_expert_range(w1_scale, lo_e, hi_e), b_microblock_size=32),
                           fused_activation=_activation(lw_local), c=h)
        mark("dispatch pull + fc1 (pipelined)")
    if plan is None:
        mark("fc1")
    with _span(gemm_timer):
        y = matmul(h, w2, lw_local.b2, a_ragged_metadata=meta_local, precision_config=pc2, gammas=gammas,
                   c=pool.ybuf)
    mark("fc2")
    pool.barrier()                                                     # every rank's expert outputs are written
    # combine: each (local token, slot) reads its row from the buffer of the rank that owns the slot's expert and
    # the k rows are summed on the fly; dropped entries (-1) stay dropped
    lo = rank * T_local * k
    comb = torch.empty(T_local * k, dtype=torch.int32, device=dev)
    _lib.check(lib.moe_ep_combine_index(_lib.ptr(md.row_sorted_indx.reshape(-1)), _lib.ptr(indx16), _lib.ptr(owner), lo,
                                        T_local * k, n, _lib.ptr(comb), _lib.stream()), "moe_ep_combine_index")
    z = torch.empty((T_local, y.shape[1]), dtype=y.dtype, device=dev)
    yptrs = (ctypes.c_void_p * W)(*pool.y_ptrs)
    _lib.check(lib.moe_gather_reduce_rows_peers(yptrs, W, n, y.stride(0), _lib.ptr(comb), T_local, k, y.shape[1],
                                                _lib.ptr(z), z.stride(0), _lib.stream()), "moe_gather_reduce_rows_peers")
    mark("output barrier + combine")
    return z


def _expert_range(t: Tensor, lo: int, hi: int) -> Tensor:
    """Experts [lo, hi) of a tiled weight tensor (the tiled layouts are expert-major: a range of experts is a range of
    the storage)."""
    from .tensor import Storage
    E = t.shape[0]
    per = t.storage.data.numel() // E
    return Tensor(Storage(t.storage.data[per * lo: per * hi], t.storage.layout), dtype=t.dtype, shape=[hi - lo] + list(t.shape[1:]))


_ep_table_cache = {}


def _ep_tables(expt_assignment, rank):
    """(local index of every expert on `rank` or -1, owner rank of every expert) as int32 device tensors, computed once
    per assignment (they are pure functions of it)."""
    key = (id(expt_assignment), rank)
    hit = _ep_table_cache.get(key)
    if hit is None or hit[0] is not expt_assignment:
        from .distributed import expert_owner
        local_expt = expt_assignment.expt_map[rank, :].to(torch.int32).contiguous()
        owner = expert_owner(expt_assignment).to(torch.int32).contiguous()
        _ep_table_cache[key] = hit = (expt_assignment, local_expt, owner)
    return hit[1], hit[2]


def moe_layer_forward_ep(x_local, logits_local, lw_local: MoeLayerWeights, k: int, expt_assignment, pool,
                         gemm_timer=None, fused_exchange=True, exchange="auto", mark=None):
    """Expert-parallel layer: tokens are sharded over ranks (x_local [T_local, d_model]), experts over ranks
    (lw_local holds this rank's experts, in increasing global id).  Routing metadata is all-gathered; token rows
    travel to the expert owners and back either through kernels that read the other ranks' peer-mapped buffers
    (the default when the pool has them) or by one NCCL all-to-all each way.

    `mark` (optional): called with a phase name after each phase has been enqueued (a benchmark records an event).
    `exchange`: "peer" (pull-dispatch / pull-combine kernels over the pool's peer-mapped buffers, see
    `SymmetricMemoryPool.enable_peer_buffers`), "nccl" (all-to-all), "auto" (peer when the pool has the buffers).
    With `fused_exchange` (NCCL form) the two GEMMs read and write the exchange buffers through index maps (fc1 gathers from
    the receive buffer, fc2 scatters into the send buffer) and the k-way combine reads the returned rows in
    place; without it the layer is the reference's composition convert_dp_to_ep -> matmul -> matmul ->
    convert_ep_to_dp -> reduce (python/triton_kernels/tests/test_distributed.py:223-247)."""
    from .distributed import (convert_dp_to_ep, convert_ep_to_dp, ep_combine_packed, ep_dispatch_packed,
                              make_exchange_plan_cuda)
    rank = pool.mesh.local_rank
    T_local = x_local.shape[0]
    peer_fit = pool.peer_ok and pool.peer_shape == (T_local, x_local.shape[1], lw_local.w2.shape[-1], k, x_local.dtype)
    if exchange == "peer" and not peer_fit:
        raise RuntimeError(f"peer exchange is not available: {pool.peer_error}")
    tokens_at = None
    if exchange in ("auto", "peer") and peer_fit:
        # this rank's tokens go into its peer-mapped buffer BEFORE the routing outputs are published: the barrier of that
        # all-gather then also tells every rank that the tokens are in place, and the dispatch needs no barrier of its own.
        # (Overwriting the buffer here is safe: every peer finished pulling the previous step's tokens before it arrived
        # at that step's last barrier.)
        if x_local.data_ptr() != pool.xbuf.data_ptr():
            pool.xbuf.copy_(x_local)
        tokens_at = getattr(pool, "n_barriers", 0)
    keep_bm, pool.gather_bitmatrix = pool.gather_bitmatrix, False     # the layer never reads the mask bits themselves
    try:
        sparse = topk(logits_local, k, apply_softmax=True, all_gather=True, symm_mem_pool=pool)
    finally:
        pool.gather_bitmatrix = keep_bm
    if mark is not None:
        mark("routing + all-gather + expert sort")
    if exchange in ("auto", "peer") and peer_fit:
        published = tokens_at is not None and getattr(pool, "n_barriers", 0) > tokens_at
        return _forward_ep_peer(x_local, sparse, lw_local, k, expt_assignment, pool, gemm_timer, mark, tokens_published=published)
    md = sparse.mask_metadata
    n_entries = md.row_sorted_indx.shape[0]
    meta_global = make_ragged_tensor_metadata(md.col_sum, n_entries)
    plan = make_exchange_plan_cuda(sparse.indx, md.col_sorted_indx, expt_assignment, pool.mesh.world_size, T_local)
    meta_local = remap_ragged_tensor_metadata(meta_global, expt_assignment.expt_map[rank, :])
    gammas = sparse.vals.reshape(-1)[md.col_sorted_indx.long().clamp_min(0)]
    pc1 = PrecisionConfig(b_mx_scale=lw_local.w1_scale, b_microblock_size=32)
    pc2 = PrecisionConfig(b_mx_scale=lw_local.w2_scale, b_microblock_size=32)
    if fused_exchange:
        recvbuf, row_of_position, n_recv = ep_dispatch_packed(x_local, k, pool, plan)
        with _span(gemm_timer):
            h = matmul(recvbuf, lw_local.w1, lw_local.b1, a_ragged_metadata=meta_local, gather_indx=row_of_position,
                       precision_config=pc1, fused_activation=_activation(lw_local))
        with _span(gemm_timer):
            y = matmul(h, lw_local.w2, lw_local.b2, a_ragged_metadata=meta_local, scatter_indx=row_of_position,
                       precision_config=pc2, gammas=gammas)
        return ep_combine_packed(y[:n_recv], k, T_local, pool, plan)
    x_ep = convert_dp_to_ep(x_local, expt_assignment, sparse.indx, md.row_sorted_indx, pool, plan=plan)
    with _span(gemm_timer):
        h = matmul(x_ep, lw_local.w1, lw_local.b1, a_ragged_metadata=meta_local, precision_config=pc1,
                   fused_activation=_activation(lw_local))
    with _span(gemm_timer):
        y = matmul(h, lw_local.w2, lw_local.b2, a_ragged_metadata=meta_local, precision_config=pc2, gammas=gammas)
    y_dp = convert_ep_to_dp(y, expt_assignment, sparse.indx, md.col_sorted_indx, pool, plan=plan)
    z, _ = reduce(y_dp.view(T_local, k, -1), dim=1)
    return z
