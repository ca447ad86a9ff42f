"""Expert parallelism: expert -> rank assignment and the two token exchanges of an EP MoE layer
(triton_kernels/distributed.py:9-95, 176-211, 256-283; distributed_details/mesh.py).

Design.  One process per GPU over `torch.distributed` (NCCL on GPUs).  Routing metadata is replicated:
every rank holds the global top-k indices and the global expert-major sort, as in the reference.  Two forms of
the exchanges:
* peer-mapped buffers (`SymmetricMemoryPool.enable_peer_buffers`): tokens, expert outputs, routing outputs and
  barrier words live in symmetric memory; the library's own kernels pull rows from the peers' buffers with plain
  loads and the barriers are kernels over the signal words, so a layer step holds no collective call;
* NCCL: each exchange is one variable-size all-to-all between a pack and an unpack kernel, with the W x W split
  sizes computed on the device from the replicated metadata and read by the host once per layer.
No TMA multicast anywhere.
"""
import ctypes
import random
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib


@dataclass
class ExptAssignment:
    # [n_shards, ceil(n_expts / 32)] int32: bit j of word j // 32 set iff expert j lives on the shard
    expt_bitmask: torch.Tensor
    # [n_shards, n_expts] bool
    expt_boolmask: torch.Tensor
    # [n_shards, n_expts] int32: local id of expert j on the shard, or -1
    expt_map: torch.Tensor
    n_expts_per_shard: list


def make_expt_dict_uniform(n_expt_shard, n_expt_tot):
    """shard i owns experts [i * (n/shards), (i+1) * (n/shards))"""
    per = n_expt_tot // n_expt_shard
    return {i: list(range(per * i, per * (i + 1))) for i in range(n_expt_shard)}


def make_expt_dict_random(n_expt_shard, n_expt_tot):
    """disjoint random subsets, no empty shard (seeded)"""
    rng = random.Random(0)
    perm = list(range(n_expt_tot))
    rng.shuffle(perm)
    cuts = [0] + sorted(rng.sample(range(1, n_expt_tot), n_expt_shard - 1)) + [n_expt_tot]
    return {i: perm[cuts[i]:cuts[i + 1]] for i in range(n_expt_shard)}


def make_expt_dict_balanced(n_expt_shard, n_expt_tot, load):
    """Equal expert counts per shard, chosen so that the measured loads (rows per expert, any sequence of numbers)
    add up as evenly as possible: heaviest expert first, each to the least loaded shard that still has room.
    (No counterpart in the reference, whose helpers place experts without looking at the router.)"""
    per = n_expt_tot // n_expt_shard
    assert per * n_expt_shard == n_expt_tot, "experts must divide evenly over the shards"
    load = [float(v) for v in load]
    assert len(load) == n_expt_tot
    owned = {i: [] for i in range(n_expt_shard)}
    total = [0.0] * n_expt_shard
    for e in sorted(range(n_expt_tot), key=lambda j: (-load[j], j)):
        shard = min((i for i in range(n_expt_shard) if len(owned[i]) < per), key=lambda i: (total[i], i))
        owned[shard].append(e)
        total[shard] += load[e]
    return {i: sorted(v) for i, v in owned.items()}


def make_expt_assignment(n_expt_shard, n_expt_tot, expt_dict, device) -> ExptAssignment:
    words = (n_expt_tot + 31) // 32
    bitmask = torch.zeros((n_expt_shard, words), dtype=torch.int64)
    boolmask = torch.zeros((n_expt_shard, n_expt_tot), dtype=torch.bool)
    counts = [0] * n_expt_tot
    for shard, experts in expt_dict.items():
        if not isinstance(experts, (list, tuple)):
            raise TypeError(f"expt_dict[{shard}] must be a list/tuple of ints")
        if len(experts) == 0:
            raise ValueError(f"shard {shard} has no experts")
        if shard < 0 or shard >= n_expt_shard:
            raise ValueError(f"shard {shard} out of range [0, {n_expt_shard})")
        for e in experts:
            if not (0 <= e < n_expt_tot):
                raise ValueError(f"expert id {e} out of range [0, {n_expt_tot})")
            counts[e] += 1
            bitmask[shard, e >> 5] |= (1 << (e & 31))
            boolmask[shard, e] = True
    if not all(c == 1 for c in counts):
        raise ValueError("each expert must be owned by exactly one shard")
    bitmask = torch.where(bitmask >= 2**31, bitmask - 2**32, bitmask).to(torch.int32)
    expt_map = torch.full((n_expt_shard, n_expt_tot), -1, dtype=torch.int32)
    for shard, experts in expt_dict.items():
        for local_id, global_id in enumerate(sorted(experts)):
            expt_map[shard, global_id] = local_id
    return ExptAssignment(bitmask.to(device), boolmask.to(device), expt_map.to(device),
                          [len(v) for v in expt_dict.values()])


MAX_PEERS = 16


class Mesh:

    def __init__(self, process_group=None):
        self.process_group = process_group
        if dist.is_available() and dist.is_initialized():
            self.world_size = dist.get_world_size(process_group)
            self.local_rank = dist.get_rank(process_group)
        else:
            self.world_size, self.local_rank = 1, 0


class SymmetricMemoryPool:
    """Process group and exchange buffers of the EP layer (the reference's pool carves one symmetric-memory arena,
    distributed.py:30-120).  `enable_peer_buffers` allocates the two exchange buffers in symmetric memory and
    learns every rank's address of them, which the pull-dispatch / push-combine kernels need; without it (or when
    the rendezvous is not available) the exchanges run as NCCL all-to-alls."""

    def __init__(self, mesh: Mesh):
        self.mesh = mesh
        self._is_initialized = False
        self.sizes = {}
        self.peer_ok = False
        self.peer_error = "enable_peer_buffers was not called"
        # the expert sort reads the gathered expert indices, not the bitmatrix: a caller that only needs the routing
        # metadata may switch the bitmatrix exchange off (the other ranks' rows of the mask are then undefined)
        self.gather_bitmatrix = True
        # expert-parallel layer over peer buffers: pull the token rows in this many groups of experts, group c + 1 on a
        # side stream under fc1 of group c (1 = one pull, then one fc1); the GEMMs of all but the last group leave
        # `overlap_idle_sms` SMs without a CTA for the pull kernel (matmul_set_idle_sms of the reference, matmul.py:239-243)
        self.overlap_chunks = 1
        self.overlap_idle_sms = 0
        self._side = {}

    def side_stream(self, device):
        key = torch.device(device).index
        if key not in self._side:
            self._side[key] = torch.cuda.Stream(device=device)
        return self._side[key]

    def enable_peer_buffers(self, n_tokens_local, d_in, d_out, k, dtype, device) -> bool:
        """x buffer [T_local, d_in] (this rank's tokens) and y buffer [T_global * k, d_out] (expert outputs in
        expert-sorted order; a rank fills the rows of its own experts) in symmetric memory; True when every rank of
        the mesh mapped every other rank's buffers."""
        ok = 1
        try:
            import torch.distributed._symmetric_memory as symm
            group = self.mesh.process_group if self.mesh.process_group is not None else dist.group.WORLD
            self.xbuf = symm.empty((n_tokens_local, d_in), dtype=dtype, device=device)
            self.ybuf = symm.empty((n_tokens_local * self.mesh.world_size * k, d_out), dtype=dtype, device=device)
            # routing outputs of this rank's tokens (top-k values fp32 + expert ids int16), and the barrier's signal words
            self.route_vals = symm.empty((n_tokens_local, k), dtype=torch.float32, device=device)
            self.route_indx = symm.empty((n_tokens_local, k), dtype=torch.int16, device=device)
            self.sig = symm.empty((MAX_PEERS,), dtype=torch.int32, device=device)
            self.sig.zero_()
            self._hx = symm.rendezvous(self.xbuf, group.group_name)
            self._hy = symm.rendezvous(self.ybuf, group.group_name)
            self._hv = symm.rendezvous(self.route_vals, group.group_name)
            self._hi = symm.rendezvous(self.route_indx, group.group_name)
            self._hs = symm.rendezvous(self.sig, group.group_name)
            self.x_ptrs = [int(p) for p in self._hx.buffer_ptrs]
            self.y_ptrs = [int(p) for p in self._hy.buffer_ptrs]
            self.rv_ptrs = [int(p) for p in self._hv.buffer_ptrs]
            self.ri_ptrs = [int(p) for p in self._hi.buffer_ptrs]
            self.sig_ptrs = [int(p) for p in self._hs.buffer_ptrs]
            assert len(self.x_ptrs) == self.mesh.world_size and all(self.x_ptrs) and all(self.y_ptrs)
            assert all(self.rv_ptrs) and all(self.ri_ptrs) and all(self.sig_ptrs)
            self._epoch = torch.zeros(1, dtype=torch.int32, device=device)
        except Exception as ex:           # no symmetric memory on this system: stay on NCCL
            ok, self.peer_error = 0, f"{type(ex).__name__}: {ex}"
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        if self.mesh.world_size > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.mesh.process_group)
        self.peer_ok = bool(int(flag.item()))
        if self.peer_ok:
            self.peer_shape = (n_tokens_local, d_in, d_out, k, dtype)
            self._barrier_word = torch.zeros(1, dtype=torch.int32, device=device)
            torch.cuda.synchronize(device)
            if self.mesh.world_size > 1:
                dist.barrier(group=self.mesh.process_group)    # every rank's signal words are zero before anyone signals
        elif ok:
            self.peer_error = "another rank could not map the buffers"
        return self.peer_ok

    def barrier(self):
        """Stream-ordered barrier over the mesh: every rank's earlier work on its current stream (peer stores
        included) is complete before any rank's later work starts."""
        if self.mesh.world_size <= 1:
            return
        self.n_barriers = getattr(self, "n_barriers", 0) + 1       # lets a caller see that a barrier followed its writes
        if self.peer_ok:
            from .matmul import _status_word
            lib = _lib.load()
            W = self.mesh.world_size
            ptrs = (ctypes.c_void_p * W)(*self.sig_ptrs)
            _lib.check(lib.moe_peer_barrier(ptrs, W, self.mesh.local_rank, _lib.ptr(self._epoch),
                                            _lib.ptr(_status_word(self._epoch.device)), _lib.stream()), "moe_peer_barrier")
        else:
            dist.all_reduce(self._barrier_word, group=self.mesh.process_group)

    def initialize_matmul(self, n_tokens_global, d_input, d_model, n_expts_act, n_expts_tot, dtype, device):
        self.sizes = dict(n_tokens_global=n_tokens_global, d_input=d_input, d_model=d_model, n_expts_act=n_expts_act,
                          n_expts_tot=n_expts_tot, dtype=dtype, device=device)
        self._is_initialized = True

    def all_gather_routing(self, y_vals, y_indx, bm_store, T_local, rank, published=False):
        """In-place all-gather of the routing outputs: rank r's rows are [r * T_local, (r+1) * T_local).  `published`:
        this rank's rows are already in the pool's peer-mapped routing buffers (the top-k kernel wrote them there)."""
        g = self.mesh.process_group
        W = self.mesh.world_size
        k = y_vals.shape[1]
        if (self.peer_ok and y_indx is not None and y_vals.dtype == torch.float32 and y_indx.dtype == torch.int16
                and self.peer_shape[0] == T_local and self.peer_shape[3] == k and y_vals.shape[0] == W * T_local
                and y_vals.is_contiguous() and y_indx.is_contiguous()):
            # no collective: publish this rank's rows in its symmetric buffers, barrier, read every rank's rows
            lib = _lib.load()
            if not published:
                self.route_vals.copy_(y_vals[rank * T_local:(rank + 1) * T_local])
                self.route_indx.copy_(y_indx[rank * T_local:(rank + 1) * T_local])
            self.barrier()
            pv = (ctypes.c_void_p * W)(*self.rv_ptrs)
            pi = (ctypes.c_void_p * W)(*self.ri_ptrs)
            _lib.check(lib.moe_allgather_peers(pv, W, T_local * k * 4, _lib.ptr(y_vals), _lib.stream()), "moe_allgather_peers")
            _lib.check(lib.moe_allgather_peers(pi, W, T_local * k * 2, _lib.ptr(y_indx), _lib.stream()), "moe_allgather_peers")
            peer_done = True
        else:
            peer_done = False
            if published:                      # the rows sit in the routing buffers only: bring them home first
                y_vals[rank * T_local:(rank + 1) * T_local].copy_(self.route_vals)
                y_indx[rank * T_local:(rank + 1) * T_local].copy_(self.route_indx)

        def gather_rows(buf):
            # byte views: NCCL has no 16-bit integer type
            full = buf[:W * T_local].view(torch.uint8)
            mine = buf[rank * T_local:(rank + 1) * T_local].view(torch.uint8).clone()
            dist.all_gather_into_tensor(full.reshape(-1), mine.reshape(-1), group=g)

        if not peer_done:
            gather_rows(y_vals)
            if y_indx is not None:
                gather_rows(y_indx)
        if not self.gather_bitmatrix:
            return
        words = bm_store.shape[0]
        loc = bm_store[:, rank * T_local:(rank + 1) * T_local].t().contiguous()      # [T_local, words]
        allr = torch.empty((W * T_local, words), dtype=bm_store.dtype, device=bm_store.device)
        dist.all_gather_into_tensor(allr, loc, group=g)
        bm_store[:, :W * T_local].copy_(allr.t())


# ---------------------------------------------------------------------------------------------------------
# exchange plan (pure index arithmetic on replicated metadata; device-agnostic so that it can be tested
# with CPU ranks)
# ---------------------------------------------------------------------------------------------------------

def expert_owner(expt_assignment: ExptAssignment) -> torch.Tensor:
    """[n_expts] int64: rank that owns each expert."""
    return expt_assignment.expt_boolmask.to(torch.int64).argmax(dim=0)


def make_exchange_plan(expt_indx, col_sorted_indx, owner, world_size, n_tokens_local):
    """For every valid expert-sorted position p: source rank s(p) (home of its token) and destination rank
    d(p) (owner of its expert).  Returns

      order   [n_valid] positions p sorted by (s, d, p)   -- the order rows travel in, on both sides
      counts  [W, W]    counts[s, d] = rows rank s sends to rank d
      flat    [n_valid] flat (token * k + slot) index of order[i]

    Rank s sends order[start(s, d) : +counts[s, d]] to d; rank d receives from s exactly that list.
    """
    k = expt_indx.shape[1]
    valid = col_sorted_indx >= 0
    p = torch.nonzero(valid).flatten()
    flat = col_sorted_indx[p].long()
    src = torch.div(flat, k * n_tokens_local, rounding_mode="floor")
    dst = owner[expt_indx.reshape(-1)[flat].long()]
    key = src * world_size + dst
    perm = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=world_size * world_size).view(world_size, world_size)
    return p[perm], counts, flat[perm]


def _starts(counts):
    c = counts.reshape(-1)
    return (torch.cumsum(c, 0) - c).view_as(counts)


@dataclass
class ExchangePlan:
    """Everything both exchanges of a layer need, computed once from the replicated routing metadata."""
    order: torch.Tensor        # [n] int32: expert-sorted positions in travel order (source, destination, position); -1 tail
    flat: torch.Tensor         # [n] int32: flat (token * k + slot) index of order[i]
    counts_host: torch.Tensor  # [W, W] int64 on the host: rows rank s sends to rank d
    starts_host: torch.Tensor  # [W, W] exclusive prefix of counts in (s, d) order


def make_exchange_plan_cuda(expt_indx, col_sorted_indx, expt_assignment, world_size, n_tokens_local) -> ExchangePlan:
    """CUDA version of `make_exchange_plan`: one key kernel, then the library's stable counting sort with
    world^2 buckets; the only host synchronisation is the read of the W x W count matrix."""
    lib = _lib.load()
    dev = col_sorted_indx.device
    k = expt_indx.shape[1]
    n = col_sorted_indx.numel()
    owner = expert_owner(expt_assignment).to(torch.int32)
    indx16 = expt_indx if expt_indx.dtype == torch.int16 else expt_indx.to(torch.int16)
    indx16 = indx16.contiguous()
    col = col_sorted_indx.reshape(-1).to(torch.int32).contiguous()
    keys = torch.empty(n, dtype=torch.int16, device=dev)
    _lib.check(lib.moe_ep_keys(_lib.ptr(col), _lib.ptr(indx16), _lib.ptr(owner), n, k * n_tokens_local, world_size,
                               _lib.ptr(keys), _lib.stream()), "moe_ep_keys")
    buckets = world_size * world_size
    counts = torch.empty(buckets, dtype=torch.int32, device=dev)
    order = torch.empty(n, dtype=torch.int32, device=dev)
    rank_of = torch.empty(n, dtype=torch.int32, device=dev)
    ws_bytes = lib.moe_bitmatrix_metadata_workspace(n, buckets, 1)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    _lib.check(lib.moe_bitmatrix_metadata(_lib.ptr(keys), 1, n, buckets, 1, None, _lib.ptr(counts), _lib.ptr(order),
                                          _lib.ptr(rank_of), _lib.ptr(ws), ws_bytes, _lib.stream()),
               "moe_bitmatrix_metadata (exchange plan)")
    flat = col[order.long().clamp_min(0)]
    counts_h = counts.cpu().to(torch.int64).view(world_size, world_size)
    return ExchangePlan(order, flat, counts_h, _starts(counts_h))


def _plan_from_torch(expt_indx, col_sorted_indx, expt_assignment, W, T_local) -> ExchangePlan:
    order, counts, flat = make_exchange_plan(expt_indx, col_sorted_indx.reshape(-1), expert_owner(expt_assignment), W, T_local)
    counts_h = counts.cpu()
    return ExchangePlan(order.to(torch.int32), flat.to(torch.int32), counts_h, _starts(counts_h))


def _rows_call(fn, src, indx, n, dst):
    row_bytes = src.shape[1] * src.element_size()
    _lib.check(fn(_lib.ptr(src), src.stride(0) * src.element_size(), _lib.ptr(indx), n, row_bytes, _lib.ptr(dst),
                  dst.stride(0) * dst.element_size(), _lib.stream()), "moe_gather_rows/moe_scatter_rows")


def _segments(plan, rank, W, column):
    """travel-order slices [start, start + count) that rank `rank` receives (column=True: from every source s)
    or holds as an expert owner; concatenated in rank order"""
    return [(int(plan.starts_host[s, rank]), int(plan.counts_host[s, rank])) for s in range(W)]


def convert_dp_to_ep(src, expt_assignment, expt_indx, gate_indx, symm_mem_pool: SymmetricMemoryPool,
                     col_sorted_indx=None, plan: ExchangePlan | None = None):
    """src [T_local, d] (this rank's tokens) -> [T_global * k, d] in global expert-sorted order, filled at
    the rows whose expert lives on this rank (other rows are left unwritten).  `gate_indx` is the global
    row_sorted_indx (flat index -> sorted position); `col_sorted_indx` (its inverse) is derived when absent.
    `plan` (from `make_exchange_plan_cuda`) is computed here when not supplied."""
    lib = _lib.load()
    mesh = symm_mem_pool.mesh
    W, rank = mesh.world_size, mesh.local_rank
    T_local, d = src.shape
    T_global, k = expt_indx.shape
    assert T_local * W <= T_global
    dev = src.device
    n = T_global * k
    if plan is None:
        if col_sorted_indx is None:
            col_sorted_indx = torch.full((n,), -1, dtype=torch.int32, device=dev)
            g = gate_indx.reshape(-1).long()
            ok = g >= 0
            col_sorted_indx[g[ok]] = torch.nonzero(ok).flatten().to(torch.int32)
        plan = make_exchange_plan_cuda(expt_indx, col_sorted_indx, expt_assignment, W, T_local)
    dst = torch.empty((n, d), dtype=src.dtype, device=dev)
    send_counts = plan.counts_host[rank].tolist()
    send_lo, n_send = int(plan.starts_host[rank, 0]), sum(send_counts)
    # pack: local token of each outgoing row, in (destination, position) order
    tok_local = torch.div(plan.flat[send_lo:send_lo + n_send], k, rounding_mode="floor") - rank * T_local
    sendbuf = torch.empty((n_send, d), dtype=src.dtype, device=dev)
    if n_send:
        _rows_call(lib.moe_gather_rows, src, tok_local.to(torch.int32), n_send, sendbuf)
    recv_counts = plan.counts_host[:, rank].tolist()
    n_recv = sum(recv_counts)
    if W > 1:
        recvbuf = torch.empty((n_recv, d), dtype=src.dtype, device=dev)
        dist.all_to_all_single(recvbuf, sendbuf, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=mesh.process_group)
    else:
        recvbuf = sendbuf
    # unpack: received row i belongs at sorted position pos[i]
    if n_recv:
        pos = torch.cat([plan.order[lo:lo + c] for lo, c in _segments(plan, rank, W, True)])
        _rows_call(lib.moe_scatter_rows, recvbuf, pos, n_recv, dst)
    return dst


def convert_ep_to_dp(src, expt_assignment, expt_indx, topk_indx, symm_mem_pool: SymmetricMemoryPool,
                     plan: ExchangePlan | None = None):
    """src [T_global * k, d] in expert-sorted order (valid at this rank's experts) -> [T_local * k, d]: row
    (t_local * k + slot) is the output of the expert in that slot.  `topk_indx` is the global
    col_sorted_indx (sorted position -> flat index)."""
    lib = _lib.load()
    mesh = symm_mem_pool.mesh
    W, rank = mesh.world_size, mesh.local_rank
    n, d = src.shape
    T_global, k = expt_indx.shape
    T_local = T_global // W
    dev = src.device
    if plan is None:
        plan = make_exchange_plan_cuda(expt_indx, topk_indx, expt_assignment, W, T_local)
    # this rank (as expert owner) returns to each home rank s the rows order[start(s, rank) : +counts[s, rank]]
    send_counts = plan.counts_host[:, rank].tolist()
    n_send = sum(send_counts)
    sendbuf = torch.empty((n_send, d), dtype=src.dtype, device=dev)
    if n_send:
        pos = torch.cat([plan.order[lo:lo + c] for lo, c in _segments(plan, rank, W, True)])
        _rows_call(lib.moe_gather_rows, src, pos, n_send, sendbuf)
    recv_counts = plan.counts_host[rank].tolist()
    n_recv = sum(recv_counts)
    if W > 1:
        recvbuf = torch.empty((n_recv, d), dtype=src.dtype, device=dev)
        dist.all_to_all_single(recvbuf, sendbuf, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=mesh.process_group)
    else:
        recvbuf = sendbuf
    dst = torch.zeros((T_local * k, d), dtype=src.dtype, device=dev)
    lo = int(plan.starts_host[rank, 0])
    if n_recv:
        where = plan.flat[lo:lo + n_recv] - rank * T_local * k
        _rows_call(lib.moe_scatter_rows, recvbuf, where.to(torch.int32), n_recv, dst)
    return dst


# ---------------------------------------------------------------------------------------------------------
# fused form used by moe_layer_forward_ep: the GEMMs read / write the exchange buffers through index maps, so
# the rows are never copied into (or out of) the [T_global * k, d] expert-sorted buffer
# ---------------------------------------------------------------------------------------------------------

def ep_dispatch_packed(src, k, symm_mem_pool: SymmetricMemoryPool, plan: ExchangePlan):
    """-> (recvbuf [n_recv, d], row_of_position [T_global * k] int32): row_of_position[p] is the row of recvbuf that
    holds the token of expert-sorted position p (-1 where p's expert lives on another rank).  Feed it to `matmul`
    as gather_indx."""
    lib = _lib.load()
    mesh = symm_mem_pool.mesh
    W, rank = mesh.world_size, mesh.local_rank
    T_local, d = src.shape
    dev = src.device
    n = plan.order.numel()
    send_counts = plan.counts_host[rank].tolist()
    send_lo, n_send = int(plan.starts_host[rank, 0]), sum(send_counts)
    tok_local = torch.div(plan.flat[send_lo:send_lo + n_send], k, rounding_mode="floor") - rank * T_local
    sendbuf = torch.empty((n_send, d), dtype=src.dtype, device=dev)
    if n_send:
        _rows_call(lib.moe_gather_rows, src, tok_local.to(torch.int32), n_send, sendbuf)
    recv_counts = plan.counts_host[:, rank].tolist()
    n_recv = sum(recv_counts)
    if W > 1:
        recvbuf = torch.empty((n_recv, d), dtype=src.dtype, device=dev)
        dist.all_to_all_single(recvbuf, sendbuf, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=mesh.process_group)
    else:
        recvbuf = sendbuf
    row_of_position = torch.full((n,), -1, dtype=torch.int32, device=dev)
    if n_recv:
        pos = torch.cat([plan.order[lo:lo + c] for lo, c in _segments(plan, rank, W, True)])
        row_of_position[pos.long()] = torch.arange(n_recv, dtype=torch.int32, device=dev)
    return recvbuf, row_of_position, n_recv


def ep_combine_packed(y_packed, k, T_local, symm_mem_pool: SymmetricMemoryPool, plan: ExchangePlan):
    """y_packed [n_recv_of_dispatch, d]: expert outputs in the row order of `ep_dispatch_packed`'s recvbuf (what
    `matmul(..., scatter_indx=row_of_position)` writes).  Sends every row home and sums the k rows of each local
    token straight out of the receive buffer.  -> [T_local, d]."""
    lib = _lib.load()
    mesh = symm_mem_pool.mesh
    W, rank = mesh.world_size, mesh.local_rank
    d = y_packed.shape[1]
    dev = y_packed.device
    send_counts = plan.counts_host[:, rank].tolist()
    recv_counts = plan.counts_host[rank].tolist()
    n_recv = sum(recv_counts)
    if W > 1:
        recvbuf = torch.empty((n_recv, d), dtype=y_packed.dtype, device=dev)
        dist.all_to_all_single(recvbuf, y_packed, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=mesh.process_group)
    else:
        recvbuf = y_packed
    lo = int(plan.starts_host[rank, 0])
    row_of_flat = torch.full((T_local * k,), -1, dtype=torch.int32, device=dev)
    if n_recv:
        where = (plan.flat[lo:lo + n_recv] - rank * T_local * k).long()
        row_of_flat[where] = torch.arange(n_recv, dtype=torch.int32, device=dev)
    z = torch.empty((T_local, d), dtype=y_packed.dtype, device=dev)
    _lib.check(lib.moe_gather_reduce_rows(_lib.ptr(recvbuf), recvbuf.stride(0), _lib.ptr(row_of_flat), T_local, k, d,
                                          _lib.ptr(z), z.stride(0), _lib.stream()), "moe_gather_reduce_rows")
    return z
