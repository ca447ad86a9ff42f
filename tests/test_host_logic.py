"""Host-side logic that needs no GPU: layouts (torch ops), block-count bounds, expert assignment, the
expert-parallel exchange plan (also across two gloo ranks), tuning constraints."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
import triton_b200
from triton_b200.distributed import make_exchange_plan, expert_owner
from triton_b200.tensor import FP4, RaggedTensorMetadata, convert_layout, wrap_torch_tensor
from triton_b200.tensor_details.layout import BlackwellMXScaleLayout, BlackwellMXValueLayout, StridedLayout


def test_n_blocks_bound_matches_oracle():
    for E in (1, 7, 128):
        for rows in (0, 1, 5, 127, 128, 129, 4096, 65536):
            for bs in (16, 32, 64, 128):
                assert RaggedTensorMetadata.n_blocks(E, rows, bs) == oracle.n_blocks(E, rows, bs)


def test_reference_layouts_round_trip_on_cpu(golden):
    g = golden("layout_bw")
    s = wrap_torch_tensor(g["scale"])
    sw = convert_layout(s, BlackwellMXScaleLayout())
    assert torch.equal(sw.storage.data, g["scale_swizzled"])
    assert torch.equal(convert_layout(sw, StridedLayout()).storage.data, g["scale"])
    v = wrap_torch_tensor(g["value"], dtype=FP4)                      # canonical: packed along N
    assert v.shape == [2, 96, 40]
    vw = convert_layout(v, BlackwellMXValueLayout())
    assert list(vw.storage.data.shape) == [2, 128, 40] and vw.storage.data.stride(-2) == 1
    assert torch.equal(vw.storage.data[:, :48], g["value_swizzled"][:, :48])
    back = convert_layout(vw, StridedLayout())
    assert torch.equal(back.storage.data, g["value"])
    # K-major strided layout (what downcast_to_mxfp produces for weights)
    km = convert_layout(v, StridedLayout(major_dim=-2))
    assert list(km.storage.data.shape) == [2, 48, 40] and km.storage.data.stride(-2) == 1
    assert torch.equal(km.storage.data, oracle.repack_fp4_oracle(g["value"], -1, -2))


def test_storage_shapes_of_reference_layouts():
    # values from the reference's tests/test_tensor.py:88-109 for the Blackwell layouts
    assert BlackwellMXValueLayout().storage_shape([3, 258, 514], True) == [3, 256, 514]
    assert BlackwellMXScaleLayout().storage_shape([3, 10, 200], False) == [1, 6, 4, 2, 256]


def test_expert_assignment():
    d = triton_b200.make_expt_dict_uniform(4, 128)
    a = triton_b200.make_expt_assignment(4, 128, d, "cpu")
    assert a.expt_boolmask.sum(0).eq(1).all() and a.n_expts_per_shard == [32] * 4
    assert a.expt_map[1, 32:64].tolist() == list(range(32)) and a.expt_map[1, 0] == -1
    assert (a.expt_bitmask[3, 3] & 0xFFFFFFFF) == 0xFFFFFFFF
    r = triton_b200.make_expt_dict_random(4, 37)
    assert sorted(sum(r.values(), [])) == list(range(37)) and all(len(v) for v in r.values())
    with pytest.raises(ValueError):
        triton_b200.make_expt_assignment(2, 4, {0: [0, 1], 1: [1, 2, 3]}, "cpu")
    assert expert_owner(a).tolist() == [e // 32 for e in range(128)]


def _plan_case(T_global=64, E=16, k=4, W=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T_global, E, generator=g)
    _, indx, _ = oracle.topk_oracle(logits, k)
    _, col, row = oracle.bitmatrix_metadata_oracle(indx, E)
    assign = triton_b200.make_expt_assignment(W, E, triton_b200.make_expt_dict_random(W, E), "cpu")
    return indx, col, row, assign


def test_exchange_plan_is_a_consistent_permutation():
    W, k = 4, 4
    indx, col, row, assign = _plan_case(W=W, k=k)
    T_local = indx.shape[0] // W
    owner = expert_owner(assign)
    order, counts, flat = make_exchange_plan(indx, col, owner, W, T_local)
    assert sorted(order.tolist()) == list(range(indx.numel()))
    assert counts.sum() == indx.numel()
    starts = (torch.cumsum(counts.reshape(-1), 0) - counts.reshape(-1)).view(W, W)
    for s in range(W):
        for d in range(W):
            seg = order[starts[s, d]:starts[s, d] + counts[s, d]]
            assert (seg[1:] > seg[:-1]).all()
            f = col[seg].long()
            assert (f // (k * T_local) == s).all()
            assert (owner[indx.reshape(-1)[f].long()] == d).all()


def _gloo_worker(rank, W, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=W)
    try:
        k, d_model = 2, 8
        indx, col, row, assign = _plan_case(T_global=32, E=8, k=k, W=W, seed=1)
        T_global = indx.shape[0]
        T_local = T_global // W
        x = torch.arange(T_global * d_model, dtype=torch.float32).view(T_global, d_model)
        owner = expert_owner(assign)
        order, counts, flat = make_exchange_plan(indx, col, owner, W, T_local)
        starts = (torch.cumsum(counts.reshape(-1), 0) - counts.reshape(-1)).view(W, W)
        # dispatch, the way convert_dp_to_ep does it, with torch indexing standing in for the CUDA row kernels
        lo, n_send = int(starts[rank, 0]), int(counts[rank].sum())
        tok = flat[lo:lo + n_send] // k
        send = x[tok]
        recv_counts = counts[:, rank].tolist()
        recv = torch.empty(sum(recv_counts), d_model)
        dist.all_to_all_single(recv, send, recv_counts, counts[rank].tolist())
        pos = torch.cat([order[int(starts[s, rank]):int(starts[s, rank]) + recv_counts[s]] for s in range(W)])
        y_ep = torch.full((T_global * k, d_model), float("nan"))
        y_ep[pos] = recv
        # what a single process would have: row p of the expert-sorted buffer is token col[p] // k
        full = x[col.long() // k]
        mine = owner[indx.reshape(-1)[col.long()].long()] == rank
        assert torch.equal(y_ep[mine], full[mine]) and torch.isnan(y_ep[~mine]).all()
        # combine back: every rank returns y_ep * 2 for the rows it owns
        send2 = (y_ep * 2)[pos]
        recv2 = torch.empty(n_send, d_model)
        dist.all_to_all_single(recv2, send2, counts[rank].tolist(), recv_counts)
        out = torch.zeros(T_local * k, d_model)
        out[flat[lo:lo + n_send] - rank * T_local * k] = recv2
        expect = (x[rank * T_local:(rank + 1) * T_local] * 2).repeat_interleave(k, 0)
        assert torch.equal(out, expect)
        ret[rank] = 1
    finally:
        dist.destroy_process_group()


def test_exchange_plan_across_two_gloo_ranks():
    W = 2
    port = 29500 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_gloo_worker, args=(r, W, port, ret)) for r in range(W)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert sorted(ret.keys()) == list(range(W))


def test_opt_flags_constraints_are_scoped():
    from triton_b200.matmul_details import opt_flags
    assert opt_flags.resolve_kernel_choice() == "auto"
    with triton_b200.scoped_opt_flags_constraints({"kernel": "simt", "block_m": 64}):
        assert opt_flags.resolve_kernel_choice() == "simt"
    assert opt_flags.resolve_kernel_choice() == "auto"
    with triton_b200.scoped_opt_flags_constraints({"split_k": 4}):
        with pytest.raises(triton_b200.InapplicableConstraint):
            opt_flags.resolve_kernel_choice()
    # a tile-shape key is honoured or refused, never dropped
    for bad in ({"block_m": 48}, {"block_k": 256}, {"is_persistent": False}, {"num_stages": 3}, {"epilogue_subtile": 2},
                {"no_such_key": 1}, {"idle_sms": -1}):
        with triton_b200.scoped_opt_flags_constraints(bad):
            with pytest.raises(triton_b200.InapplicableConstraint):
                opt_flags.resolve_kernel_choice()
    with triton_b200.scoped_opt_flags_constraints({"block_m": 32, "block_n": 384, "block_k": 128, "split_k": 1,
                                                   "is_persistent": True, "num_stages": None, "idle_sms": 8}):
        assert opt_flags.resolve_kernel_choice() == "auto"
        assert opt_flags.resolve_tile_m() == 32 and opt_flags.resolve_tile_n() == 384 and opt_flags.get_idle_sms() == 8
    assert opt_flags.get_idle_sms() == 0


def test_balanced_expert_placement():
    """Equal counts per shard, every expert placed once, and a far better balance than contiguous blocks on a skewed load."""
    import random
    from triton_b200.distributed import make_expt_dict_balanced, make_expt_dict_uniform
    rng = random.Random(0)
    load = [2.718 ** rng.gauss(0, 1) for _ in range(128)]
    for shards in (2, 4, 8):
        d = make_expt_dict_balanced(shards, 128, load)
        assert sorted(e for v in d.values() for e in v) == list(range(128))
        assert all(len(v) == 128 // shards for v in d.values())
        spread = lambda dd: max(sum(load[e] for e in v) for v in dd.values()) / (sum(load) / shards)
        assert spread(d) < 1.02 <= spread(make_expt_dict_uniform(shards, 128)) + 1e-9 or spread(d) < 1.02
        assert spread(d) <= spread(make_expt_dict_uniform(shards, 128))


def test_shuffled_value_layout_matches_reference_fixture(golden):
    """BlackwellMX4ValueShuffledLayout against the reference's own output (two tilings, K and N both padded)."""
    from triton_b200.tensor_details.layout import BlackwellMX4ValueShuffledLayout
    g = golden("layout_bw2")
    v = wrap_torch_tensor(g["value"], dtype=FP4)                      # canonical [E, K, N/2]
    assert v.shape == [2, 200, 300]
    for (bk, bn), key in (((128, 256), "value_shuffled_128_256"), ((64, 128), "value_shuffled_64_128")):
        lay = BlackwellMX4ValueShuffledLayout(block_k=bk, block_n=bn)
        sw = convert_layout(v, lay)
        assert list(sw.storage.data.shape) == list(g[key].shape)
        assert torch.equal(sw.storage.data, g[key])
        assert torch.equal(convert_layout(sw, StridedLayout()).storage.data, g["value"])
    # the reference's storage-shape known answers (tests/test_tensor.py:99-100, 103-105)
    from triton_b200.tensor_details.layout import BlackwellActMXScaleLayout
    assert BlackwellMX4ValueShuffledLayout().make_transformation([3, 258, 514], True).storage_shape == [3, 4, 3, 256, 64]
    assert BlackwellMX4ValueShuffledLayout().make_transformation([0, 64], True).storage_shape == [1, 0, 1, 256, 64]
    assert BlackwellActMXScaleLayout(None).make_transformation([130, 65], False).storage_shape == [1, 2, 18, 2, 256]
    assert BlackwellActMXScaleLayout(None).make_transformation([3, 130, 65], False).storage_shape == [1, 6, 18, 2, 256]
    assert BlackwellActMXScaleLayout(None).make_transformation([0, 64], False).storage_shape == [1, 0, 16, 2, 256]


def test_act_scale_layout_matches_reference_fixture_and_oracle(golden):
    from triton_b200.tensor_details.layout import BlackwellActMXScaleLayout
    g = golden("layout_bw2")
    a = wrap_torch_tensor(g["act_scale"])
    sw = convert_layout(a, BlackwellActMXScaleLayout(None))
    assert torch.equal(sw.storage.data, g["act_scale_swizzled"])
    assert torch.equal(convert_layout(sw, StridedLayout()).storage.data, g["act_scale"])
    # ragged: every slice starts at a new block of 128 rows; rows past the slices are dropped
    sizes = torch.tensor([130, 0, 5, 128, 20], dtype=torch.int32)
    M = int(sizes.sum()) + 17
    gen = torch.Generator().manual_seed(4)
    s = torch.randint(0, 255, (M, 12), generator=gen, dtype=torch.uint8)
    offs = torch.zeros(6, dtype=torch.int32)
    offs[1:] = torch.cumsum(sizes, 0)
    nb = [[0] * 6 for _ in range(4)]
    for b, bs in enumerate((16, 32, 64, 128)):
        run = 0
        for e in range(5):
            nb[b][e] = run
            run += (int(sizes[e]) + bs - 1) // bs
        nb[b][5] = run
    md = RaggedTensorMetadata(sizes, offs, torch.tensor(nb, dtype=torch.int32),
                              torch.zeros((4, RaggedTensorMetadata.max_n_blocks(5, M)), dtype=torch.int32))
    lay = BlackwellActMXScaleLayout(md)
    sw = convert_layout(wrap_torch_tensor(s), lay)
    assert torch.equal(sw.storage.data, oracle.swizzle_act_mx_scale_oracle(s, sizes.tolist()))
    back = convert_layout(sw, StridedLayout()).storage.data
    assert torch.equal(back[: int(sizes.sum())], s[: int(sizes.sum())]) and not back[int(sizes.sum()):].any()


def test_default_weight_layout_arguments():
    from triton_b200.tensor_details.layout import (B200MXScaleLayout, B200MXValueLayout, make_default_matmul_mxfp4_w_layout,
                                                   make_default_matmul_mxfp4_w_scale_layout)
    assert isinstance(make_default_matmul_mxfp4_w_layout(mx_axis=-2, allow_blackwell_value_shuffle=True), B200MXValueLayout)
    assert isinstance(make_default_matmul_mxfp4_w_scale_layout(mx_axis=1), B200MXScaleLayout)
    with pytest.raises(NotImplementedError):
        make_default_matmul_mxfp4_w_layout(mx_axis=-1)


def test_weight_file_round_trip_on_cpu(tmp_path):
    """save_layer_weights / load_layer_weights: every tensor comes back byte for byte, in the layout it was saved in."""
    from triton_b200.moe import MoeLayerWeights
    from triton_b200.tensor import Storage, Tensor
    from triton_b200.tensor_details.layout import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout, B200MXScaleLayout,
                                                   B200MXValueLayout)
    from triton_b200.weights_io import load_layer_weights, read_header, save_layer_weights
    g = torch.Generator().manual_seed(0)
    E, K, N = 3, 256, 384

    def tiled(layout, logical, nbytes, fp4):
        data = torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8)
        return Tensor(Storage(data, layout), dtype=FP4 if fp4 else triton_b200.tensor.UINT8, shape=logical)

    nv, ns = E * 2 * 3 * 8192, E * 2 * 3 * 512
    lw = MoeLayerWeights(tiled(B200MXValueLayout(), [E, K, N], nv, True), tiled(B200MXScaleLayout(), [E, K // 32, N], ns, False),
                         torch.randn(E, N, generator=g).bfloat16(),
                         tiled(B200MXValueLayout(), [E, N // 2, K], E * 2 * 2 * 8192, True),
                         tiled(B200MXScaleLayout(), [E, N // 64, K], E * 2 * 2 * 512, False),
                         torch.randn(E, K, generator=g).bfloat16(), alpha=1.5, limit=None,
                         w1_bs=tiled(B200BlockScaledValueLayout(), [E, K, N], nv, True),
                         w1_bs_scale=tiled(B200BlockScaledScaleLayout(), [E, K // 32, N], ns, False))
    path = tmp_path / "layer.moeb200w"
    size = save_layer_weights(path, lw)
    assert path.stat().st_size == size and size % 4096 == 0
    hdr = read_header(path)
    assert all(e["offset"] % 4096 == 0 for e in hdr["tensors"].values()) and "w2_bs" not in hdr["tensors"]
    back = load_layer_weights(path, "cpu")
    assert back.alpha == 1.5 and back.limit is None and back.w2_bs is None
    for name in ("w1", "w1_scale", "w2", "w2_scale", "w1_bs", "w1_bs_scale"):
        a, b = getattr(lw, name), getattr(back, name)
        assert type(a.storage.layout) is type(b.storage.layout) and a.shape == b.shape and a.dtype == b.dtype
        assert torch.equal(a.storage.data, b.storage.data)
    assert torch.equal(lw.b1, back.b1) and torch.equal(lw.b2, back.b2)
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"not a weight file at all")
    with pytest.raises(ValueError):
        read_header(bad)
