#!/usr/bin/env python
"""Benchmark of the MoE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T]

A step is one MoE layer forward (routing -> fc1 + SwiGLU -> fc2 x routing weight -> k-way combine; with
N > 1 ranks also the two expert-parallel all-to-all exchanges) over one batch of seeded synthetic input of
the gpt-oss-120b layer shape: d_model 2880, d_ff 2880 (fused gate+up 5760), 128 experts, top-4, bf16
activations N(0,1), MXFP4 weights from bf16 N(0,0.02), router logits fp32 N(0,1) plus a per-expert bias
N(0,1) (skewed load), 16384 tokens per rank (weak scaling).  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU restatement of the reference's torch implementation (oracle/) on the host
cores of this box on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

D_MODEL, D_FF, N_EXPTS, TOP_K = 2880, 2880, 128, 4
FLOP_PER_ROW_FC1 = 2 * D_MODEL * 2 * D_FF          # 33,177,600
FLOP_PER_ROW_FC2 = 2 * D_FF * D_MODEL              # 16,588,800
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def workload_name(tokens_per_rank, n_gpus):
    return (f"gpt-oss-{'120b' if N_EXPTS == 128 else ('20b' if N_EXPTS == 32 else 'like')} MoE layer: d_model {D_MODEL}, fused gate+up {2 * D_FF}, E={N_EXPTS} top-{TOP_K}, "
            f"{tokens_per_rank} tokens/rank, skewed router, bf16 x MXFP4, EP over {n_gpus} GPU(s)")


# ---------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"gpu_idle": 0x1, "applications_clocks_setting": 0x2, "sw_power_cap": 0x4, "hw_slowdown": 0x8,
                 "sync_boost": 0x10, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "display_clock_setting": 0x100}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                except Exception:
                    pass
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "power_w_max": (max(self.power) if self.power else None)}


# ---------------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (a port of the reference's torch implementation) on a bounded sample
# ---------------------------------------------------------------------------------------------------------
CPU_SAMPLE_TOKENS, CPU_SAMPLE_EXPTS = 256, 8


def cpu_sample_inputs(seed=0):
    import oracle
    g = torch.Generator().manual_seed(seed)
    E, T = CPU_SAMPLE_EXPTS, CPU_SAMPLE_TOKENS
    x = torch.randn(T, D_MODEL, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g) + torch.randn(E, generator=g)
    w1 = (torch.randn(E, D_MODEL, 2 * D_FF, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(E, D_FF, D_MODEL, generator=g) * 0.02).bfloat16()
    q1, s1 = oracle.downcast_to_mxfp_oracle(w1, 1)
    q2, s2 = oracle.downcast_to_mxfp_oracle(w2, 1)
    b1 = (torch.randn(E, 2 * D_FF, generator=g) * 0.01).bfloat16()
    b2 = (torch.randn(E, D_MODEL, generator=g) * 0.01).bfloat16()
    return x, logits, (q1, s1, b1, q2, s2, b2)


def cpu_layer_step(x, logits, w):
    """One layer the way the reference's torch path runs it: weights are dequantised inside every call
    (matmul.py:772-817 is invoked by matmul_torch)."""
    import oracle
    q1, s1, b1, q2, s2, b2 = w
    w1 = oracle.dequant_weight_oracle(q1, s1)
    w2 = oracle.dequant_weight_oracle(q2, s2)
    return oracle.moe_layer_oracle(x, logits, w1, b1, w2, b2, TOP_K, 1.702, 7.0)


def cpu_sample_desc():
    return (f"{CPU_SAMPLE_TOKENS} tokens, top-{TOP_K} over {CPU_SAMPLE_EXPTS} experts of the same shape "
            f"(d_model {D_MODEL}, fused gate+up {2 * D_FF}), weights dequantised per call as the reference does")


def run_cpu_baseline(steps, warmup):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, logits, w = cpu_sample_inputs()
    for _ in range(warmup):
        cpu_layer_step(x, logits, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_layer_step(x, logits, w)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return CPU_SAMPLE_TOKENS / dt, dt, cores


def reference_arm(args, rank):
    if rank != 0:
        return
    steps, warmup = min(args.steps, 10), min(args.warmup, 2)
    v, dt, cores = run_cpu_baseline(steps, warmup)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.tokens, args.gpus), "timed": "CPU oracle on a bounded sample"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_desc()},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def gemm_traffic_note():
    """DRAM bytes per launch of the grouped-GEMM kernel from the committed ncu summary, if one exists."""
    p = ROOT / "profiles" / "gemm_tc_traffic.json"
    if p.exists():
        try:
            return json.loads(p.read_text())
        except Exception:
            return None
    return None


def micro_bench(args):
    """Standalone routing / MXFP4 quantiser timings against the measured copy bandwidth.

    Every timed call runs after a 512 MB write that evicts its inputs from L2; the time is the mean of per-call CUDA
    event pairs.  Bytes are algorithmic: what the operator must read and write once."""
    import triton_b200 as tb
    from triton_b200.numerics_details.mxfp import downcast_to_mxfp, upcast_from_mxfp
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        ts = []
        for _ in range(args.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sum(ts) / len(ts)

    out = {"micro": args.micro, "steps": args.steps, "l2": "flushed by a 512 MB write before every timed call",
           "peak_gbs": peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth", "kernels": {}}

    def add(name, ms, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["kernels"][name] = {"ms": ms, "algorithmic_bytes": nbytes, "gbs": gbs, "frac": gbs / peaks["hbm_gbs"]}

    if args.micro == "routing":
        T, E, k = 16384, N_EXPTS, TOP_K
        logits = torch.randn(T, E, device=dev, generator=g)
        sp = tb.topk(logits, k)
        add("topk [16384,128] fp32 -> top-4 values, indices, bitmatrix", timed(lambda: tb.topk(logits, k)),
            T * E * 4 + T * k * (4 + 2) + T * (E // 8))
        add("routing (topk + expert sort + ragged metadata)", timed(lambda: tb.routing(logits, k)),
            T * E * 4 + T * k * (4 + 2) + T * (E // 8) + T * k * (2 + 4 + 4) + E * 4 * 12)
    else:
        R = C = 8192
        x = torch.randn(R, C, device=dev, generator=g)
        x = torch.where(torch.rand(R, C, device=dev, generator=g) < 0.01, x * 100, x).bfloat16()
        q, sc = downcast_to_mxfp(x, torch.uint8, axis=1)
        add("downcast_to_mxfp bf16 [8192,8192] axis 1", timed(lambda: downcast_to_mxfp(x, torch.uint8, axis=1)),
            R * C * 2 + R * C // 2 + R * C // 32)
        add("upcast_from_mxfp -> bf16 [8192,8192] axis 1", timed(lambda: upcast_from_mxfp(q, sc, torch.bfloat16, axis=1)),
            R * C * 2 + R * C // 2 + R * C // 32)
        q0, sc0 = downcast_to_mxfp(x, torch.uint8, axis=0)
        add("downcast_to_mxfp bf16 [8192,8192] axis 0 (strided)", timed(lambda: downcast_to_mxfp(x, torch.uint8, axis=0)),
            R * C * 2 + R * C // 2 + R * C // 32)
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per rank")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="expert-parallel exchange: kernels over peer-mapped buffers, or NCCL all-to-all")
    ap.add_argument("--no-graph", action="store_true", help="never replay the step from a CUDA graph")
    ap.add_argument("--experts", type=int, default=128, help="experts of the layer (32: the gpt-oss-20b shape)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "tcgen05", "tcgen05-pair", "stream"],
                    help="pin the grouped-GEMM kernel (default: the library's choice)")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "uniform"],
                    help="expert placement over ranks: equal counts balanced by measured load, or contiguous blocks")
    ap.add_argument("--micro", default=None, choices=["routing", "mxfp"],
                    help="time the memory-bound kernels on their standalone configuration instead of the layer")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    global N_EXPTS
    N_EXPTS = args.experts
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.micro:
        if rank == 0:
            micro_bench(args)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")

    import torch.distributed as dist
    import triton_b200 as tb
    from triton_b200.moe import moe_layer_forward, moe_layer_forward_ep
    from triton_b200.testing import make_synthetic_layer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    if args.kernel != "auto":
        tb.update_opt_flags_constraints({"kernel": args.kernel})
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    T = args.tokens
    E_local = N_EXPTS // world
    # every rank builds its own experts with a rank-dependent seed; router bias and tokens are seeded per rank
    # decode-sized steps run on the block-scaled kernel, which streams its own copy of the weights
    lw = make_synthetic_layer(E_local, D_MODEL, D_FF, dev, seed=1000 + rank, block_scaled=(T <= 1024))
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(T, D_MODEL, device=dev, generator=g).bfloat16()
    gb = torch.Generator(device=dev).manual_seed(12345)
    expert_bias = torch.randn(N_EXPTS, device=dev, generator=gb)
    logits = torch.randn(T, N_EXPTS, device=dev, generator=g) + expert_bias
    pool = assignment = None
    if world > 1:
        if args.placement == "balanced":
            # one calibration batch: rows per expert over all ranks' tokens, then equal-count placement by load (the
            # weights are synthetic per rank, so placing an expert only decides which logits column it answers to)
            load = tb.topk(logits, TOP_K).mask_metadata.col_sum.to(torch.float32)
            dist.all_reduce(load)
            expt_dict = tb.make_expt_dict_balanced(world, N_EXPTS, load.cpu().tolist())
        else:
            expt_dict = tb.make_expt_dict_uniform(world, N_EXPTS)
        assignment = tb.make_expt_assignment(world, N_EXPTS, expt_dict, dev)
        pool = tb.SymmetricMemoryPool(tb.Mesh(dist.group.WORLD))
        pool.initialize_matmul(T * world, D_MODEL, D_MODEL, TOP_K, N_EXPTS, torch.bfloat16, dev)
        if args.exchange != "nccl":
            pool.enable_peer_buffers(T, D_MODEL, D_MODEL, TOP_K, torch.bfloat16, dev)

    # decode sizes on one GPU: the step is replayed from a CUDA graph (a dozen short launches per step cost more host
    # time than GPU time; at prefill sizes a replayed step was no faster than eager launches and its static output
    # serialises the host-streaming pipeline); the roofline pass below times the GEMM launches of the eager step
    graphed, graph_note = None, None
    if world == 1 and T <= 1024 and not args.no_graph:
        from triton_b200.moe import GraphedMoeLayer
        graphed = GraphedMoeLayer(lw, TOP_K, T, D_MODEL, N_EXPTS, dev)

    if world > 1 and pool.peer_ok and args.exchange != "nccl" and not args.no_graph:
        # over peer buffers the expert-parallel step holds no collective call and no host synchronisation either:
        # replay it from a graph, too (every rank takes the same branch)
        from triton_b200.moe import GraphedMoeLayer
        graphed = GraphedMoeLayer(lw, TOP_K, T, D_MODEL, N_EXPTS, dev, forward=lambda xi, li: moe_layer_forward_ep(
            xi, li, lw, TOP_K, assignment, pool, exchange=args.exchange))

    def step(xi, li, timer=None):
        if graphed is not None and timer is None:
            return graphed(xi, li)
        if world > 1:
            return moe_layer_forward_ep(xi, li, lw, TOP_K, assignment, pool, gemm_timer=timer, exchange=args.exchange)
        return moe_layer_forward(xi, li, lw, TOP_K, gemm_timer=timer)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        z = step(x, logits)
    barrier()
    tb.matmul_check_status()

    # ---- timed region: K steps, inputs resident in HBM; the expert weights (1.69 GB / world) are far larger
    # than the 126 MB L2 and are streamed once per step, so no separate L2 flush is needed -----------------
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev[0].record()
        for _ in range(args.steps):
            z = step(x, logits)
        ev[1].record()
        barrier()
    elapsed_ms = ev[0].elapsed_time(ev[1])
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    tb.matmul_check_status()
    ms_per_step = elapsed_ms / args.steps
    value = T * world / (ms_per_step * 1e-3)

    # ---- the dominant kernel, timed on its own stream position inside the same step --------------------
    # (events around the two grouped-GEMM launches of each step; every other kernel of the step still runs)
    class GemmTimer:
        def __init__(self):
            self.spans = []

        def __call__(self):
            return self

        def __enter__(self):
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e0.record()

        def __exit__(self, *a):
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.spans.append((self._e0, e1))
            return False

    gt = GemmTimer()
    barrier()
    for _ in range(args.steps):
        # a spin kernel ahead of every step lets the host enqueue the whole step before the GPU reaches it, so that the
        # spans hold GPU time only (no launch gaps)
        torch.cuda._sleep(int(2.0e6 if T > 1024 else 4.0e5))
        z = step(x, logits, gt)
    barrier()
    # per-step sum of the spans, median over the steps (a span stretches when the host falls behind the GPU)
    per_call = [e0.elapsed_time(e1) for e0, e1 in gt.spans]
    calls_per_step = max(1, len(per_call) // args.steps)
    per_step = sorted(sum(per_call[i:i + calls_per_step]) for i in range(0, len(per_call), calls_per_step))
    gemm_ms = [per_step[len(per_step) // 2] * args.steps]
    n_gemm = [len(gt.spans)]
    rows_local = T * TOP_K                        # routed rows this rank multiplies (average under uniform ownership)
    flop_per_step = rows_local * (FLOP_PER_ROW_FC1 + FLOP_PER_ROW_FC2)
    gemm_ms_per_step = gemm_ms[0] / args.steps
    achieved_tflops = flop_per_step / (gemm_ms_per_step * 1e-3) / 1e12
    peaks = measured_peaks()
    traffic = gemm_traffic_note()
    # weight streaming: bytes of the experts that received at least one row (W1 + S1 + W2 + S2 + biases), per step
    sp = tb.topk(logits, TOP_K) if world == 1 else None
    if sp is not None:
        n_active = int((sp.mask_metadata.col_sum > 0).sum().item())
    else:
        n_active = E_local
    bytes_per_expert = (D_MODEL * 2 * D_FF + D_FF * D_MODEL) // 2 + (D_MODEL * 2 * D_FF + D_FF * D_MODEL) // 32 + \
        (2 * D_FF + D_MODEL) * 2
    act_bytes = rows_local * (D_MODEL * 2 + D_FF * 2 * 2 + D_MODEL * 2)
    stream_gbs = (n_active * bytes_per_expert + act_bytes) / (gemm_ms_per_step * 1e-3) / 1e9
    roofline = {
        "bound": "tensor", "kernel": "gemm_tc_kernel (fc1 + fc2 launches of a step, bf16 kind::f16 after in-SM dequant)",
        "achieved": achieved_tflops, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
        "frac": achieved_tflops / peaks["bf16_tflops_sustained"], "peak_source": f"{peaks['source']} bf16 cuBLAS, sustained",
        "traffic": None if traffic is None else traffic.get("dram_bytes_per_step"),
        "ms_per_step_in_kernel": gemm_ms_per_step, "launches_per_step": n_gemm[0] / args.steps,
        "frac_of_inferred_mxfp4_peak": achieved_tflops / (4 * peaks["bf16_tflops_sustained"]),
        "hbm": {"active_experts": n_active, "algorithmic_gbs": stream_gbs, "peak_gbs": peaks["hbm_gbs"],
                "frac": stream_gbs / peaks["hbm_gbs"]},
    }
    if T <= 256:        # decode regime: the grouped GEMM streams weights, HBM is the bound
        if graphed is not None:
            # the eager GEMM spans include launch gaps that the replayed graph does not have: charge the weight bytes
            # to the whole graph step instead (routing and combine included, so this understates the kernel)
            stream_gbs = (n_active * bytes_per_expert + act_bytes) / (ms_per_step * 1e-3) / 1e9
            roofline["hbm"].update({"algorithmic_gbs": stream_gbs, "frac": stream_gbs / peaks["hbm_gbs"]})
            roofline["kernel"] = "gemm_stream_kernel (fc1 + fc2), timed as the whole replayed step"
        roofline.update({"bound": "hbm", "achieved": stream_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": stream_gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
                         "tflops": achieved_tflops})

    # ---- end to end: host buffers in, host result out, through the public API ---------------------------
    e2e = None
    if not args.no_e2e:
        xh = x.cpu().pin_memory()
        lh = logits.cpu().pin_memory()
        zh = [torch.empty((T, D_MODEL), dtype=torch.bfloat16).pin_memory() for _ in range(2)]

        def e2e_time(run, n):
            run(3)
            barrier()
            ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev2[0].record()
            run(n)
            ev2[1].record()
            barrier()
            t2 = torch.tensor([ev2[0].elapsed_time(ev2[1])], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t2, op=dist.ReduceOp.MAX)
            return float(t2.item()) / n

        n_e2e = max(4, args.steps // 2)
        # host buffers in, host buffers out, through the package's streaming front end: every step uploads its inputs
        # and downloads its result; uploads / downloads of neighbouring steps overlap the compute of this one
        from triton_b200.moe import HostStreamingLayer
        pipe = HostStreamingLayer(lambda xd, ld: step(xd, ld), T, D_MODEL, N_EXPTS, dev)

        def run_pipelined(n):
            for i in range(n):
                pipe.submit(xh, lh, zh[i & 1])
            pipe.drain()

        xd, ld = torch.empty_like(x), torch.empty_like(logits)

        def run_serial(n):                      # one stream: upload, compute, download, one step after the other
            for i in range(n):
                xd.copy_(xh, non_blocking=True)
                ld.copy_(lh, non_blocking=True)
                zh[i & 1].copy_(step(xd, ld), non_blocking=True)

        try:
            ms_e2e, how = e2e_time(run_pipelined, n_e2e), "upload, compute and download of consecutive steps overlap (3 streams)"
        except Exception as ex:                 # keep the line: fall back to the plain single-stream sequence
            torch.cuda.synchronize()
            ms_e2e, how = e2e_time(run_serial, n_e2e), f"single stream (pipelined front end failed: {type(ex).__name__})"
        e2e = {"value": T * world / (ms_e2e * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": xh.numel() * 2 + lh.numel() * 4, "d2h_bytes_per_step": zh[0].numel() * 2,
               "steps": n_e2e, "pipelined": how}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, dt, cores = run_cpu_baseline(3, 1)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_desc(),
                        "s_per_step": dt}

    launches_per_step = 9 if world == 1 else 16     # topk, 3 sort passes, ragged, row gather, 2 GEMMs, reduce (+ exchange plan, remap, row moves)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(T, world),
                       "cuda_graph": graphed is not None if graph_note is None else graph_note,
                       "expert_placement": None if world == 1 else
                       (f"{E_local} per rank, balanced by measured load" if args.placement == "balanced" else "contiguous blocks"),
                       "exchange": None if world == 1 else ("peer-mapped buffers" if pool.peer_ok else
                                                            f"NCCL all-to-all ({pool.peer_error})"),
                       "l2": "inputs larger than L2 (weights streamed once per step)",
                       "tflops_per_step_algorithmic": flop_per_step * world / 1e12 if world > 1 else flop_per_step / 1e12},
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline, "cpu_baseline": cpu_baseline,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
