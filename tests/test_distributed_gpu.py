"""Expert-parallel MoE layer on 2, 4 or 8 GPUs, one process per GPU over NCCL, against the single-GPU layer: the eager
step with every exchange form, then the step replayed from a CUDA graph on two further inputs (the reference's
tests/test_distributed.py:306-342 compares the same pairs, graph replay included)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, n_tokens, d_model, d_ff, n_expts, k, mode, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import oracle
        import triton_b200 as tb
        from triton_b200.moe import MoeLayerWeights, moe_layer_forward, moe_layer_forward_ep
        from triton_b200.testing import make_synthetic_layer
        from triton_b200.tensor import FP4, convert_layout, wrap_torch_tensor
        from triton_b200.tensor_details.layout import (B200BlockScaledScaleLayout, B200BlockScaledValueLayout,
                                                       B200MXScaleLayout, B200MXValueLayout)
        torch.manual_seed(0)
        lw = make_synthetic_layer(n_expts, d_model, d_ff, dev, seed=0, keep_canonical=True)     # same on every rank
        x = torch.randn(n_tokens, d_model, device=dev).bfloat16()
        logits = torch.randn(n_tokens, n_expts, device=dev)
        z_ref = moe_layer_forward(x, logits, lw, k)
        expt_dict = (tb.make_expt_dict_uniform if mode == "uniform" else tb.make_expt_dict_random)(world, n_expts)
        assign = tb.make_expt_assignment(world, n_expts, expt_dict, dev)
        mine = assign.expt_boolmask[rank]

        def shard(q, s, vl=B200MXValueLayout, sl_=B200MXScaleLayout):
            tq = convert_layout(wrap_torch_tensor(q[mine].transpose(1, 2).contiguous().transpose(1, 2), dtype=FP4), vl())
            ts = convert_layout(wrap_torch_tensor(s[mine].transpose(1, 2).contiguous().transpose(1, 2)), sl_())
            return tq, ts

        w1, s1 = shard(lw.w1_q, lw.w1_s)
        w2, s2 = shard(lw.w2_q, lw.w2_s)
        lw_local = MoeLayerWeights(w1, s1, lw.b1[mine].contiguous(), w2, s2, lw.b2[mine].contiguous())
        # the block-scaled copy too: steps with few rows per expert run on it
        lw_local.w1_bs, lw_local.w1_bs_scale = shard(lw.w1_q, lw.w1_s, B200BlockScaledValueLayout, B200BlockScaledScaleLayout)
        lw_local.w2_bs, lw_local.w2_bs_scale = shard(lw.w2_q, lw.w2_s, B200BlockScaledValueLayout, B200BlockScaledScaleLayout)
        ret[f"block_scaled{rank}"] = lw_local.use_block_scaled(n_tokens * k // world)
        pool = tb.SymmetricMemoryPool(tb.Mesh(dist.group.WORLD))
        pool.initialize_matmul(n_tokens, d_model, d_model, k, n_expts, torch.bfloat16, dev)
        T_local = n_tokens // world
        sl = slice(rank * T_local, (rank + 1) * T_local)
        # the reference's composition, the fused NCCL exchange twice, then the peer-memory exchange twice
        variants = [("nccl", False), ("nccl", True), ("nccl", True)]
        if pool.enable_peer_buffers(T_local, d_model, d_model, k, torch.bfloat16, dev):
            variants += [("peer", True), ("peer", True)]
        ret[f"peer{rank}"] = pool.peer_ok or pool.peer_error
        for exchange, fused in variants:
            z_loc = moe_layer_forward_ep(x[sl].contiguous(), logits[sl].contiguous(), lw_local, k, assign, pool,
                                         fused_exchange=fused, exchange=exchange)
            tb.matmul_check_status()
            z_all = torch.empty_like(z_ref)
            dist.all_gather_into_tensor(z_all, z_loc)
            oracle.assert_close_oracle(z_ref.cpu(), z_all.cpu(), maxtol=2e-2, rmstol=4e-3,
                                       what=f"EP ({exchange}, fused={fused}) vs single GPU")
        if pool.peer_ok:
            # the dispatch pull in groups of experts on a side stream, overlapped with fc1 of the previous group
            for chunks, idle in ((2, 0), (3, 8)):
                pool.overlap_chunks, pool.overlap_idle_sms = chunks, idle
                z_loc = moe_layer_forward_ep(x[sl].contiguous(), logits[sl].contiguous(), lw_local, k, assign, pool, exchange="peer")
                tb.matmul_check_status()
                z_all = torch.empty_like(z_ref)
                dist.all_gather_into_tensor(z_all, z_loc)
                oracle.assert_close_oracle(z_ref.cpu(), z_all.cpu(), maxtol=2e-2, rmstol=4e-3,
                                           what=f"EP (peer, {chunks} overlapped groups) vs single GPU")
            pool.overlap_chunks, pool.overlap_idle_sms = 2, 0          # the replayed step below keeps one overlapped form
            # what the benchmark times: the collective-free step captured once and replayed on new inputs
            from triton_b200.moe import GraphedMoeLayer
            gl = GraphedMoeLayer(lw_local, k, T_local, d_model, n_expts, dev, forward=lambda xi, li: moe_layer_forward_ep(
                xi, li, lw_local, k, assign, pool, exchange="peer"))
            for seed in (11, 12):
                g2 = torch.Generator(device=dev).manual_seed(seed)               # the same batch on every rank
                x2 = torch.randn(n_tokens, d_model, device=dev, generator=g2).bfloat16()
                l2 = torch.randn(n_tokens, n_expts, device=dev, generator=g2)
                z_ref2 = moe_layer_forward(x2, l2, lw, k)
                z_loc = gl(x2[sl].contiguous(), l2[sl].contiguous())
                tb.matmul_check_status()
                z_all = torch.empty_like(z_ref2)
                dist.all_gather_into_tensor(z_all, z_loc)
                oracle.assert_close_oracle(z_ref2.cpu(), z_all.cpu(), maxtol=2e-2, rmstol=4e-3,
                                           what=f"EP graph replay (seed {seed}) vs single GPU")
            ret[f"graph{rank}"] = True
        ret[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n_tokens, d_model, d_ff, n_expts, k, mode", [
    (16, 64, 64, 4, 4, "uniform"),
    (128, 512, 256, 16, 4, "random"),
    (64, 2880, 2880, 32, 4, "random"),            # decode-sized: few rows per expert, the block-scaled kernel
    (4096, 2880, 2880, 128, 4, "uniform"),
])
def test_expert_parallel_layer_matches_single_gpu(world, n_tokens, d_model, d_ff, n_expts, k, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if n_expts % world or n_tokens % world:
        pytest.skip("experts / tokens do not divide over the ranks")
    port = 29700 + (os.getpid() + world * 7 + n_tokens) % 2000
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_tokens, d_model, d_ff, n_expts, k, mode, ret))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    codes = [p.exitcode for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    assert codes == [0] * world, codes
    assert sorted(k for k in ret.keys() if isinstance(k, int)) == list(range(world))
    print("peer exchange:", {k: v for k, v in ret.items() if not isinstance(k, int)})


@pytest.mark.parametrize("T_global, E, k, W", [(64, 16, 4, 4), (4096, 128, 4, 8), (1000, 37, 2, 2)])
def test_cuda_exchange_plan_equals_torch_plan(T_global, E, k, W):
    """The CUDA plan (key kernel + counting sort) against the index arithmetic written with torch ops."""
    import triton_b200 as tb
    from triton_b200.distributed import expert_owner, make_exchange_plan, make_exchange_plan_cuda
    dev = "cuda"
    torch.manual_seed(T_global)
    logits = torch.randn(T_global, E, device=dev)
    sp = tb.topk(logits, k)
    col = sp.mask_metadata.col_sorted_indx
    assign = tb.make_expt_assignment(W, E, tb.make_expt_dict_random(W, E), dev)
    T_local = T_global // W
    plan = make_exchange_plan_cuda(sp.indx, col, assign, W, T_local)
    order, counts, flat = make_exchange_plan(sp.indx, col.long(), expert_owner(assign), W, T_local)
    n = order.numel()
    assert torch.equal(plan.order[:n].long(), order) and (plan.order[n:] == -1).all()
    assert torch.equal(plan.flat[:n].long(), flat)
    assert torch.equal(plan.counts_host, counts.cpu())
