#!/usr/bin/env python
"""Benchmark of the MoE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T]

A step is one MoE layer forward (routing -> fc1 + SwiGLU -> fc2 x routing weight -> k-way combine; with
N > 1 ranks also the two expert-parallel exchanges) over one batch of seeded synthetic input of the
gpt-oss-120b layer shape: d_model 2880, d_ff 2880 (fused gate+up 5760), 128 experts, top-4, bf16
activations N(0,1), MXFP4 weights from bf16 N(0,0.02), router logits fp32 N(0,1) plus a per-expert bias
N(0,1) (skewed load), 16384 tokens per rank (weak scaling).  Rank 0 prints ONE JSON line.

Beside the headline the line carries
  parity      the layer output of sampled tokens against the CPU oracle, for the eager and the replayed step
  blocks      the K-step timed block repeated (median / min / max) and one pass of >= 2 s (sustained clocks)
  roofline    the grouped-GEMM launches against the measured bf16 peak (burst for the short block, sustained
              for the long pass), and weight streaming against the measured copy bandwidth
  decode      the same layer at 1 / 4 / 16 / 64 tokens (GEMM launches alone and whole replayed step)
  sweep_20b   the gpt-oss-20b shape (32 experts) at 1 .. 16384 tokens
  micro       routing [16384, 128] and the MXFP4 quantiser [8192, 8192]
  cpu_baseline the CPU oracle on the reference's CPU-sized layer, on the routing / quantiser case and on a bounded
              sample of this workload

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
BYTES_PER_EXPERT = (D_MODEL * 2 * D_FF + D_FF * D_MODEL) // 2 + (D_MODEL * 2 * D_FF + D_FF * D_MODEL) // 32 + \
    (2 * D_FF + D_MODEL) * 2                       # W1 + W2 packed, their scales, both biases (bf16): 13,236,480
ALPHA, LIMIT = 1.702, 7.0
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def workload_name(tokens_per_rank, n_gpus, n_expts=None):
    e = N_EXPTS if n_expts is None else n_expts
    return (f"gpt-oss-{'120b' if e == 128 else ('20b' if e == 32 else 'like')} MoE layer: d_model {D_MODEL}, fused gate+up {2 * D_FF}, E={e} top-{TOP_K}, "
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
# CPU baselines: the oracle (a port of the reference's torch implementation) on the host cores
# ---------------------------------------------------------------------------------------------------------
CPU_SAMPLE_TOKENS, CPU_SAMPLE_EXPTS = 256, 8


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.lower().startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def _timed_cpu(fn, runs, warm=1):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(runs):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[len(ts) // 2]


def _cpu_layer_inputs(T, E, d, ff, k, seed=0, skew=False):
    import oracle
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g)
    if skew:
        logits = logits + torch.randn(E, generator=g)
    w1 = (torch.randn(E, d, 2 * ff, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(E, ff, d, generator=g) * 0.02).bfloat16()
    q1, s1 = oracle.downcast_to_mxfp_oracle(w1, 1)
    q2, s2 = oracle.downcast_to_mxfp_oracle(w2, 1)
    b1 = (torch.randn(E, 2 * ff, generator=g) * 0.01).bfloat16()
    b2 = (torch.randn(E, d, generator=g) * 0.01).bfloat16()
    return x, logits, (q1, s1, b1, q2, s2, b2)


def cpu_layer_step(x, logits, w, k):
    """One layer the way the reference's torch path runs it: weights are dequantised inside every call
    (matmul.py:772-817 is invoked by matmul_torch)."""
    import oracle
    q1, s1, b1, q2, s2, b2 = w
    w1 = oracle.dequant_weight_oracle(q1, s1)
    w2 = oracle.dequant_weight_oracle(q2, s2)
    return oracle.moe_layer_oracle(x, logits, w1, b1, w2, b2, k, ALPHA, LIMIT)


def cpu_sample_desc():
    return (f"{CPU_SAMPLE_TOKENS} tokens, top-{TOP_K} over {CPU_SAMPLE_EXPTS} experts of the same shape "
            f"(d_model {D_MODEL}, fused gate+up {2 * D_FF}), weights dequantised per call as the reference does")


def run_cpu_sample(steps, warmup, threads=None):
    cores = threads or (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    x, logits, w = _cpu_layer_inputs(CPU_SAMPLE_TOKENS, CPU_SAMPLE_EXPTS, D_MODEL, D_FF, TOP_K, skew=True)
    dt = _timed_cpu(lambda: cpu_layer_step(x, logits, w, TOP_K), steps, warmup)
    return CPU_SAMPLE_TOKENS / dt, dt, cores


def run_cpu_c1(threads):
    """The reference's own CPU-sized case: one layer, 256 tokens, d_model 512, d_ff 1024, 8 experts top-2."""
    torch.set_num_threads(threads)
    x, logits, w = _cpu_layer_inputs(256, 8, 512, 1024, 2, seed=0)
    dt = _timed_cpu(lambda: cpu_layer_step(x, logits, w, 2), 5, 1)
    return {"tokens_per_s": 256 / dt, "s_per_step": dt, "threads": threads}


def run_cpu_c2(threads):
    """Routing on [16384, 128] logits top-4 and the MXFP4 quantiser on bf16 [8192, 8192] (1 % outliers x 100), the
    quantiser in chunks of 1024 rows to bound its fp32 temporaries."""
    import oracle
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(16384, 128, generator=g)

    def route():
        vals, indx, _ = oracle.topk_oracle(logits, 4, apply_softmax=True)
        col_sum, col_sorted, row_sorted = oracle.bitmatrix_metadata_oracle(indx, 128)
        oracle.ragged_metadata_oracle(col_sum, 16384 * 4)

    t_route = _timed_cpu(route, 3, 1)
    R = C = 8192
    x = torch.randn(R, C, generator=g)
    x = torch.where(torch.rand(R, C, generator=g) < 0.01, x * 100, x).bfloat16()
    chunks = [x[i:i + 1024] for i in range(0, R, 1024)]
    t0 = time.perf_counter()
    qs = [oracle.downcast_to_mxfp_oracle(c, -1) for c in chunks]
    t_down = time.perf_counter() - t0
    t0 = time.perf_counter()
    for q, s in qs:
        oracle.upcast_from_mxfp_oracle(q, s, torch.bfloat16, -1)
    t_up = time.perf_counter() - t0
    nbytes = R * C * 2 + R * C // 2 + R * C // 32
    return {"threads": threads, "routing_s": t_route, "routing_tokens_per_s": 16384 / t_route,
            "downcast_s": t_down, "downcast_gbs": nbytes / t_down / 1e9, "upcast_s": t_up, "upcast_gbs": nbytes / t_up / 1e9,
            "note": "quantiser run in 8 chunks of 1024 rows"}


def cpu_baseline_record(sample_steps=3, full=True):
    cores = os.cpu_count() or 1
    v, dt, _ = run_cpu_sample(sample_steps, 1)
    rec = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_desc(), "s_per_step": dt,
           "cpu_model": cpu_model(), "torch": torch.__version__}
    if full:
        rec["c1_reference_cpu_case"] = {"config": "T=256, d_model 512, d_ff 1024 (fused 2048), E=8 top-2, seed 0",
                                        "all_cores": run_cpu_c1(cores), "one_thread": run_cpu_c1(1)}
        rec["c2_routing_quantiser"] = run_cpu_c2(cores)
        torch.set_num_threads(cores)
    return rec


def reference_arm(args, rank):
    if rank != 0:
        return
    steps, warmup = min(args.steps, 10), min(args.warmup, 2)
    v, dt, cores = run_cpu_sample(steps, warmup)
    cb = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_desc(), "cpu_model": cpu_model()}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.tokens, args.gpus), "timed": "CPU oracle on a bounded sample"},
        "cpu_baseline": cb,
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ---------------------------------------------------------------------------------------------------------
# GPU arm: helpers
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


def gemm_traffic_note(tokens, n_expts, world):
    """DRAM bytes per step of the grouped-GEMM launches from the committed ncu summary; only for the configuration the
    summary was scaled to."""
    p = ROOT / "profiles" / "gemm_tc_traffic.json"
    if not p.exists():
        return None
    try:
        d = json.loads(p.read_text())
    except Exception:
        return None
    if world == 1 and d.get("tokens") == tokens and d.get("experts") == n_expts:
        return d.get("dram_bytes_per_step")
    return None


def median(v):
    s = sorted(v)
    return s[len(s) // 2]


def launch_count():
    from triton_b200 import _lib
    return int(_lib.load().moe_launch_count())


class Spans:
    """CUDA-event pairs around chosen launches of a step (`with spans():`)."""

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

    def per_step_ms(self, steps):
        per_call = [e0.elapsed_time(e1) for e0, e1 in self.spans]
        c = max(1, len(per_call) // max(steps, 1))
        return [sum(per_call[i:i + c]) for i in range(0, len(per_call), c)], c


def slice_experts(lw, n):
    """The first n experts of a layer as a layer of its own (the tiled layouts are expert-major, so a prefix of the
    storage is the layer of a prefix of the experts)."""
    from triton_b200.moe import MoeLayerWeights
    from triton_b200.tensor import Storage, Tensor
    E = lw.n_expts

    def cut(t):
        if t is None:
            return None
        per = t.storage.data.numel() // E
        shape = [n] + list(t.shape[1:])
        return Tensor(Storage(t.storage.data[:per * n], t.storage.layout), dtype=t.dtype, shape=shape)

    return MoeLayerWeights(cut(lw.w1), cut(lw.w1_scale), lw.b1[:n], cut(lw.w2), cut(lw.w2_scale), lw.b2[:n], lw.alpha,
                           lw.limit, w1_bs=cut(lw.w1_bs), w1_bs_scale=cut(lw.w1_bs_scale), w2_bs=cut(lw.w2_bs),
                           w2_bs_scale=cut(lw.w2_bs_scale))


def make_batch(T, n_expts, dev, seed, expert_bias):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(T, D_MODEL, device=dev, generator=g).bfloat16()
    logits = torch.randn(T, n_expts, device=dev, generator=g) + expert_bias[:n_expts]
    return x, logits


# ---------------------------------------------------------------------------------------------------------
# parity of what is timed: sampled tokens of rank 0 against the CPU oracle
# ---------------------------------------------------------------------------------------------------------
def parity_record(z_by_name, x, logits, lw, world, assignment, dev, n_sample=8):
    """`z_by_name`: {"eager": z, "graph": z, ...} outputs [T, d_model] of rank 0's step on (x, logits).  The oracle
    recomputes `n_sample` token rows from the canonical MXFP4 weights of the experts they hit (at N > 1 the owners'
    weights are regenerated here from their seeds)."""
    import oracle
    from triton_b200.testing import make_synthetic_layer
    T = x.shape[0]
    rows = sorted(set(int(i) for i in torch.linspace(0, T - 1, n_sample).round().tolist()))
    ridx = torch.tensor(rows, device=dev)
    xs, ls = x[ridx].cpu(), logits[ridx].cpu()
    layers = {0: lw}
    E_local = lw.n_expts

    def locate(e):
        if world == 1:
            return 0, e
        col = assignment.expt_map[:, e]
        r = int((col >= 0).nonzero()[0, 0])
        return r, int(col[r])

    def expert_weights(e):
        r, j = locate(e)
        if r not in layers:
            # another rank's experts: the same generator and seed as that rank used
            layers[r] = make_synthetic_layer(E_local, D_MODEL, D_FF, dev, seed=1000 + r, keep_canonical=True, layouts=False)
        L = layers[r]
        w1 = oracle.dequant_weight_oracle(L.w1_q[j:j + 1].cpu(), L.w1_s[j:j + 1].cpu())[0]
        w2 = oracle.dequant_weight_oracle(L.w2_q[j:j + 1].cpu(), L.w2_s[j:j + 1].cpu())[0]
        return w1, L.b1[j].cpu(), w2, L.b2[j].cpu()

    torch.set_num_threads(os.cpu_count() or 1)
    ref = oracle.moe_layer_tokens_oracle(xs, ls, expert_weights, TOP_K, ALPHA, LIMIT)
    out = {"tokens": len(rows), "rows": rows, "oracle": "oracle.moe_layer_tokens_oracle on canonical MXFP4 weights",
           "tolerance": {"rel_l2": 1e-2, "max_rel": 3e-2}, "ok": True}
    for name, z in z_by_name.items():
        got = z[ridx].cpu()
        rel = oracle.rel_l2(ref, got)
        mx, _ = oracle.rel_errors(ref, got)
        ok = bool(rel < 1e-2 and mx <= 3e-2)
        out[name] = {"rel_l2": float(rel), "max_rel": float(mx), "ok": ok}
        out["ok"] = out["ok"] and ok
    return out


# ---------------------------------------------------------------------------------------------------------
# sub-records (1 GPU): decode, 20b sweep, memory-bound micro-benchmarks
# ---------------------------------------------------------------------------------------------------------
def _graph_of(fn, dev, warm=2):
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    return g, out


def _time_replays(graphs, rounds):
    for g in graphs:
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        for g in graphs:
            g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (rounds * len(graphs))


def decode_point(lw, n_expts, T, dev, expert_bias, peaks, n_batches=6, rounds=5):
    """One token count of the decode regime.  `n_batches` different batches are replayed round-robin, so that a replay
    does not find the previous replay's experts in L2 (at one token a step touches only 4 experts = 53 MB)."""
    import triton_b200 as tb
    from triton_b200.matmul import PrecisionConfig, matmul
    from triton_b200.moe import GraphedMoeLayer, _activation
    keep, g_gemm, g_step, n_act = [], [], [], []
    for b in range(n_batches):
        x, logits = make_batch(T, n_expts, dev, 7000 + 100 * T + b, expert_bias)
        ragged, gi, si, sp = tb.routing(logits, TOP_K)
        n_act.append(int((sp.mask_metadata.col_sum > 0).sum().item()))
        gam = sp.vals.reshape(-1)[si.long()].contiguous()
        w1, s1, w2, s2 = lw.fc_weights(T * TOP_K)
        pc1 = PrecisionConfig(b_mx_scale=s1, b_microblock_size=32)
        pc2 = PrecisionConfig(b_mx_scale=s2, b_microblock_size=32)

        def gemms(x=x, ragged=ragged, gi=gi, si=si, gam=gam, w1=w1, w2=w2, pc1=pc1, pc2=pc2):
            h = matmul(x, w1, lw.b1, ragged, gather_indx=gi, precision_config=pc1, fused_activation=_activation(lw))
            return matmul(h, w2, lw.b2, ragged, scatter_indx=si, precision_config=pc2, gammas=gam)

        g, y = _graph_of(gemms, dev)
        g_gemm.append(g)
        layer = GraphedMoeLayer(lw, TOP_K, T, D_MODEL, n_expts, dev, warmup=2)
        layer.x.copy_(x)
        layer.logits.copy_(logits)
        g_step.append(layer.graph)
        keep.append((x, logits, ragged, gi, si, sp, gam, y, layer, pc1, pc2))     # everything a graph reads stays alive
    ms_gemm = _time_replays(g_gemm, rounds)
    ms_step = _time_replays(g_step, rounds)
    act = sum(n_act) / len(n_act)
    wbytes = act * BYTES_PER_EXPERT
    return {"tokens": T, "active_experts": act, "weight_mb": wbytes / 1e6,
            "kernel": "gemm_mx_kernel (block-scaled)" if lw.use_block_scaled(T * TOP_K) else "bf16 kernels",
            "gemm_ms": ms_gemm, "gemm_gbs": wbytes / ms_gemm / 1e6, "gemm_frac_hbm": wbytes / ms_gemm / 1e6 / peaks["hbm_gbs"],
            "step_ms": ms_step, "step_gbs": wbytes / ms_step / 1e6, "step_frac_hbm": wbytes / ms_step / 1e6 / peaks["hbm_gbs"],
            "tokens_per_s": T / (ms_step * 1e-3)}


def decode_record(lw, dev, expert_bias, peaks):
    pts = [decode_point(lw, N_EXPTS, T, dev, expert_bias, peaks) for T in (1, 4, 16, 64)]
    return {"what": "gpt-oss-120b layer, 1 GPU, CUDA-graph replays over 6 rotating batches (weights of consecutive "
                    "replays differ, L2 does not hold them); gemm_* = the fc1 + fc2 launches alone (with their token "
                    "packing), step_* = the whole layer step; GB/s = bytes of the active experts' weights / time",
            "peak_gbs": peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth", "points": pts}


def sweep_20b_record(lw20, dev, expert_bias, peaks):
    import triton_b200 as tb
    from triton_b200.moe import moe_layer_forward
    pts = []
    for T in (1, 16, 64, 512, 4096, 16384):
        if T <= 1024:
            p = decode_point(lw20, 32, T, dev, expert_bias, peaks, n_batches=4)
            rec = {"tokens": T, "ms_per_step": p["step_ms"], "tokens_per_s": p["tokens_per_s"], "cuda_graph": True,
                   "gemm_ms": p["gemm_ms"], "active_experts": p["active_experts"], "kernel": p["kernel"]}
            flop = T * TOP_K * (FLOP_PER_ROW_FC1 + FLOP_PER_ROW_FC2)
            if T >= 512:
                tf = flop / (p["gemm_ms"] * 1e-3) / 1e12
                rec.update({"gemm_tflops": tf, "gemm_frac_bf16_burst": tf / peaks["bf16_tflops"]})
            else:
                rec.update({"gemm_gbs": p["gemm_gbs"], "gemm_frac_hbm": p["gemm_frac_hbm"]})
        else:
            x, logits = make_batch(T, 32, dev, 9000 + T, expert_bias)
            for _ in range(3):
                moe_layer_forward(x, logits, lw20, TOP_K)
            torch.cuda.synchronize()
            sp = Spans()
            n = 8
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                moe_layer_forward(x, logits, lw20, TOP_K, gemm_timer=sp)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / n
            per_step, _ = sp.per_step_ms(n)
            gm = median(per_step)
            tf = T * TOP_K * (FLOP_PER_ROW_FC1 + FLOP_PER_ROW_FC2) / (gm * 1e-3) / 1e12
            rec = {"tokens": T, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "cuda_graph": False, "gemm_ms": gm,
                   "gemm_tflops": tf, "gemm_frac_bf16_burst": tf / peaks["bf16_tflops"], "kernel": "gemm_tc_kernel (bf16)"}
        pts.append(rec)
    tb.matmul_check_status()
    return {"what": "gpt-oss-20b layer shape (E=32 top-4, d_model 2880, fused gate+up 5760), 1 GPU, whole layer step",
            "points": pts}


def tensor_roof_record(dev):
    """Tensor-pipe roofs measured by this repository's own issue-loop kernel (operands resident in shared memory,
    one CTA per SM): what a kernel of that MMA kind can reach at most on this GPU at the clocks of this run."""
    import ctypes
    from triton_b200 import _lib
    lib = _lib.load()
    names = {0: "bf16 kind::f16", 1: "e4m3 kind::f8f6f4", 2: "e2m1 x e4m3 block-scaled kind::mxf8f6f4", 3: "e2m1 x e2m1 block-scaled kind::mxf4"}
    out = {"how": "moe_tensor_roof: 148 CTAs x 4000 x 4 back-to-back tcgen05.mma M128 N256, best of 5, CUDA events", "tflops": {}}
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for kind, name in names.items():
        flop = ctypes.c_double(0.0)
        best = None
        for _ in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(lib.moe_tensor_roof(kind, 4000, ctypes.byref(flop), _lib.ptr(status), _lib.stream()), "moe_tensor_roof")
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        out["tflops"][name] = flop.value / (best * 1e-3) / 1e12
    out["status"] = int(status.item())
    return out


def act_fp8_record(lw, dev, expert_bias, peaks, T, n_steps, roofs):
    """The same layer in the reference's fp8 mode: e4m3 tokens, e4m3 between the two GEMMs, both GEMMs on the block-scaled
    kernel (kind::mxf8f6f4, weights straight into the MMA).  Parity against the oracle fed the same quantised rows."""
    import oracle
    import triton_b200 as tb
    from triton_b200.moe import moe_layer_forward
    x, logits = make_batch(T, N_EXPTS, dev, 0, expert_bias)
    x8 = x.to(torch.float8_e4m3fn)
    for _ in range(3):
        z = moe_layer_forward(x8, logits, lw, TOP_K)
    torch.cuda.synchronize()
    tb.matmul_check_status()
    sp = Spans()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_steps):
        moe_layer_forward(x8, logits, lw, TOP_K, gemm_timer=sp)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n_steps
    per_step, _ = sp.per_step_ms(n_steps)
    gm = median(per_step)
    tf = T * TOP_K * (FLOP_PER_ROW_FC1 + FLOP_PER_ROW_FC2) / (gm * 1e-3) / 1e12
    rows = sorted(set(int(i) for i in torch.linspace(0, T - 1, 8).round().tolist()))
    ridx = torch.tensor(rows, device=dev)

    def expert_weights(e):
        w1 = oracle.dequant_weight_oracle(lw.w1_q[e:e + 1].cpu(), lw.w1_s[e:e + 1].cpu())[0]
        w2 = oracle.dequant_weight_oracle(lw.w2_q[e:e + 1].cpu(), lw.w2_s[e:e + 1].cpu())[0]
        return w1, lw.b1[e].cpu(), w2, lw.b2[e].cpu()

    ref = oracle.moe_layer_tokens_oracle(x8[ridx].cpu().float(), logits[ridx].cpu(), expert_weights, TOP_K, ALPHA, LIMIT,
                                         h_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16)
    got = z[ridx].cpu()
    rel = oracle.rel_l2(ref, got)
    mx, _ = oracle.rel_errors(ref, got)
    roof = roofs["tflops"].get("e2m1 x e4m3 block-scaled kind::mxf8f6f4") if roofs else None
    return {"what": "e4m3 activations x MXFP4 weights, gemm_mx_kernel (kind::mxf8f6f4) for fc1 and fc2, eager steps",
            "tokens": T, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "gemm_ms_per_step": gm, "gemm_tflops": tf,
            "frac_of_measured_mxf8f6f4_roof": None if not roof else tf / roof,
            "parity": {"tokens": len(rows), "rel_l2": float(rel), "max_rel": float(mx), "ok": bool(rel < 1e-2 and mx <= 3e-2),
                       "oracle": "moe_layer_tokens_oracle on the same e4m3 inputs, e4m3 between the GEMMs"}}


def micro_record(dev, peaks, steps=5):
    """Standalone routing / MXFP4 quantiser timings against the measured copy bandwidth.  Every timed call runs
    after a 512 MB write that evicts its inputs from L2 and a short spin kernel that lets the host enqueue the call
    ahead of the GPU; the time is the median of per-call CUDA event pairs.  Bytes are algorithmic: what the operator must
    read and write once."""
    import triton_b200 as tb
    from triton_b200.numerics_details.mxfp import downcast_to_mxfp, upcast_from_mxfp
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)

    def timed(fns):
        """`fns`: the same call on several distinct inputs.  One event pair spans all of them, issued back to back after
        the flush, so each runs on cold data while the span holds no launch latency between kernels."""
        for fn in fns:
            fn()
        ts, launches = [], 0
        for _ in range(steps):
            flush.fill_(1)
            torch.cuda._sleep(400000)          # the host enqueues the calls while the GPU spins
            l0 = launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for fn in fns:
                fn()
            e1.record()
            torch.cuda.synchronize()
            launches = (launch_count() - l0) // len(fns)
            ts.append(e0.elapsed_time(e1) / len(fns))
        return median(ts), launches

    # a write-dominated kernel cannot reach the copy bandwidth (half reads, half writes): measure the pure-write rate too
    big = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    fill_ms = []
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        big.zero_()
        e1.record()
        torch.cuda.synchronize()
        fill_ms.append(e0.elapsed_time(e1))
    write_gbs = (1 << 30) / (min(fill_ms[2:]) * 1e-3) / 1e9
    del big
    out = {"l2": "flushed by a 512 MB write before every timed span; a span is the same call on 4 distinct inputs, back to back",
           "peak_gbs": peaks["hbm_gbs"],
           "peak_source": f"{peaks['source']} copy bandwidth", "write_only_gbs": write_gbs,
           "write_only_source": "torch zero_ of 1 GiB, best of 4, measured in this run", "kernels": {}}

    def add(name, res, nbytes):
        ms, launches = res
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["kernels"][name] = {"ms": ms, "launches": launches, "algorithmic_bytes": nbytes, "gbs": gbs,
                                "frac": gbs / peaks["hbm_gbs"]}

    T, E, k = 16384, 128, TOP_K
    NV = 4
    lgs = [torch.randn(T, E, device=dev, generator=g) for _ in range(NV)]
    add("topk [16384,128] fp32 -> top-4 values, indices, bitmatrix", timed([lambda l=l: tb.topk(l, k) for l in lgs]),
        T * E * 4 + T * k * (4 + 2) + T * (E // 8))
    add("routing (topk + expert sort + ragged metadata)", timed([lambda l=l: tb.routing(l, k) for l in lgs]),
        T * E * 4 + T * k * (4 + 2) + T * (E // 8) + T * k * (2 + 4 + 4) + E * 4 * 12)
    # the router: logits = x @ Wg + bg and the top-k in one kernel, against the two steps apart (library GEMM + topk)
    K = D_MODEL
    rx = [torch.randn(T, K, device=dev, generator=g).bfloat16() for _ in range(NV)]
    wg = tb.prepare_router_weight((torch.randn(K, E, device=dev, generator=g) / K ** 0.5).bfloat16())
    wg_rows = wg.contiguous()
    bg = torch.randn(E, device=dev, generator=g)
    bgb = bg.bfloat16()
    r_bytes = T * K * 2 + K * E * 2 + T * k * (2 + 2) + T * (E // 8)
    add("router_topk fused [16384,2880] x [2880,128] -> top-4", timed([lambda x=x: tb.router_topk(x, wg, bg, k) for x in rx]), r_bytes)
    add("router as two steps: library GEMM (bf16 logits) + topk",
        timed([lambda x=x: tb.topk(torch.addmm(bgb, x, wg_rows), k) for x in rx]), r_bytes + 2 * T * E * 2)
    for name in ("router_topk fused [16384,2880] x [2880,128] -> top-4", "router as two steps: library GEMM (bf16 logits) + topk"):
        out["kernels"][name]["note"] = "includes the three expert-sort launches that build the SparseMatrix metadata"
    rx64 = [x[:64].contiguous() for x in rx]
    add("router_topk fused, 64 tokens", timed([lambda x=x: tb.router_topk(x, wg, bg, k) for x in rx64]), 64 * K * 2 + K * E * 2)
    add("router as two steps, 64 tokens", timed([lambda x=x: tb.topk(torch.addmm(bgb, x, wg_rows), k) for x in rx64]), 64 * K * 2 + K * E * 2)
    del rx, rx64
    R = C = 8192
    xs = []
    for _ in range(NV):
        x = torch.randn(R, C, device=dev, generator=g)
        xs.append(torch.where(torch.rand(R, C, device=dev, generator=g) < 0.01, x * 100, x).bfloat16())
    del x
    qs = [downcast_to_mxfp(x, torch.uint8, axis=1) for x in xs]
    nb = R * C * 2 + R * C // 2 + R * C // 32
    add("downcast_to_mxfp bf16 [8192,8192] axis 1", timed([lambda x=x: downcast_to_mxfp(x, torch.uint8, axis=1) for x in xs]), nb)
    add("upcast_from_mxfp -> bf16 [8192,8192] axis 1",
        timed([lambda q=q, sc=sc: upcast_from_mxfp(q, sc, torch.bfloat16, axis=1) for q, sc in qs]), nb)
    up = out["kernels"]["upcast_from_mxfp -> bf16 [8192,8192] axis 1"]
    # 79 % of the dequantiser's bytes are writes: its bound is the time to write R * C * 2 bytes at the write-only rate
    up["write_bound_ms"] = R * C * 2 / write_gbs / 1e6
    up["frac_of_write_bound"] = up["write_bound_ms"] / up["ms"]
    add("downcast_to_mxfp bf16 [8192,8192] axis 0 (strided)",
        timed([lambda x=x: downcast_to_mxfp(x, torch.uint8, axis=0) for x in xs]), nb)
    return out


# ---------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per rank")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="skip the decode / 20b sweep / micro sub-records")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--blocks", type=int, default=10, help="repetitions of the K-step timed block")
    ap.add_argument("--sustained-s", type=float, default=2.0, help="length of the back-to-back pass (0: skip)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="expert-parallel exchange: kernels over peer-mapped buffers, or NCCL all-to-all")
    ap.add_argument("--no-graph", action="store_true", help="never replay the step from a CUDA graph")
    ap.add_argument("--experts", type=int, default=128, help="experts of the layer (32: the gpt-oss-20b shape)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "tcgen05", "tcgen05-pair", "stream", "mx"],
                    help="pin the grouped-GEMM kernel (default: the library's choice)")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "uniform"],
                    help="expert placement over ranks: equal counts balanced by measured load, or contiguous blocks")
    ap.add_argument("--ep-chunks", type=int, default=1,
                    help="expert-parallel layer: pull the token rows in this many expert groups, overlapped with fc1")
    ap.add_argument("--ep-idle-sms", type=int, default=0, help="SMs the overlapped fc1 launches leave to the pull kernel")
    ap.add_argument("--micro", default=None, choices=["routing", "mxfp", "all"],
                    help="print only the memory-bound micro-benchmarks")
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
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")

    import torch.distributed as dist
    import triton_b200 as tb
    from triton_b200.moe import GraphedMoeLayer, moe_layer_forward, moe_layer_forward_ep
    from triton_b200.testing import make_synthetic_layer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks = measured_peaks()
    if args.micro:
        if rank == 0:
            print(json.dumps({"micro": micro_record(dev, peaks, steps=max(args.steps // 4, 5))}), flush=True)
        return
    if args.kernel != "auto":
        tb.update_opt_flags_constraints({"kernel": args.kernel})
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    T = args.tokens
    E_local = N_EXPTS // world
    want_sub = world == 1 and not args.no_sub and T == 16384 and N_EXPTS == 128 and args.kernel == "auto"
    want_decode_ep = world > 1 and not args.no_sub and T == 16384
    # every rank builds its own experts with a rank-dependent seed; router bias and tokens are seeded per rank.  The
    # canonical (packed, K-contiguous) weights are kept for the parity check; decode-sized steps run on the block-scaled
    # kernel, which streams its own copy of the weights
    lw = make_synthetic_layer(E_local, D_MODEL, D_FF, dev, seed=1000 + rank, keep_canonical=not args.no_parity,
                              block_scaled=(T <= 1024 or want_sub or want_decode_ep) and args.kernel in ("auto", "mx"))
    gb = torch.Generator(device=dev).manual_seed(12345)
    expert_bias = torch.randn(N_EXPTS, device=dev, generator=gb)
    x, logits = make_batch(T, N_EXPTS, dev, rank, expert_bias)
    pool = assignment = None
    placement_note = None
    if world > 1:
        if args.placement == "balanced":
            # placement calibrated on a batch of its own (another seed than any timed batch): rows per expert over all
            # ranks' calibration tokens, then equal-count placement by load
            _, cal_logits = make_batch(T, N_EXPTS, dev, 500000 + rank, expert_bias)
            load = tb.topk(cal_logits, TOP_K).mask_metadata.col_sum.to(torch.float32)
            dist.all_reduce(load)
            expt_dict = tb.make_expt_dict_balanced(world, N_EXPTS, load.cpu().tolist())
            placement_note = f"{E_local} per rank, balanced by the load of a separate calibration batch"
        else:
            expt_dict = tb.make_expt_dict_uniform(world, N_EXPTS)
            placement_note = "contiguous blocks"
        assignment = tb.make_expt_assignment(world, N_EXPTS, expt_dict, dev)
        pool = tb.SymmetricMemoryPool(tb.Mesh(dist.group.WORLD))
        pool.initialize_matmul(T * world, D_MODEL, D_MODEL, TOP_K, N_EXPTS, torch.bfloat16, dev)
        if args.exchange != "nccl":
            pool.enable_peer_buffers(T, D_MODEL, D_MODEL, TOP_K, torch.bfloat16, dev)
        pool.overlap_chunks, pool.overlap_idle_sms = args.ep_chunks, args.ep_idle_sms

    def eager(xi, li, timer=None, mark=None):
        if world > 1:
            return moe_layer_forward_ep(xi, li, lw, TOP_K, assignment, pool, gemm_timer=timer, exchange=args.exchange, mark=mark)
        return moe_layer_forward(xi, li, lw, TOP_K, gemm_timer=timer)

    # decode sizes on one GPU, and the collective-free expert-parallel step over peer buffers: replayed from a CUDA graph
    graphed = None
    use_graph = not args.no_graph and ((world == 1 and T <= 1024) or (world > 1 and pool.peer_ok and args.exchange != "nccl"))
    l0 = launch_count()
    z_eager = eager(x, logits)
    launches_per_step = launch_count() - l0      # a replayed graph launches the same kernels as the step it captured
    if use_graph:
        graphed = GraphedMoeLayer(lw, TOP_K, T, D_MODEL, N_EXPTS, dev, forward=lambda xi, li: eager(xi, li))

    def step(xi, li, timer=None):
        if graphed is not None and timer is None:
            return graphed(xi, li)
        return eager(xi, li, timer)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        z = step(x, logits)
    barrier()
    tb.matmul_check_status()

    # ---- parity of what is timed (outside the timed region) ------------------------------------------------
    parity = None
    if not args.no_parity:
        zs = {"eager": z_eager}
        if graphed is not None:
            zs["graph"] = step(x, logits)
        barrier()
        if rank == 0:
            parity = parity_record(zs, x, logits, lw, world, assignment, dev)
        barrier()

    # ---- timed region: blocks of K steps, inputs resident in HBM; the expert weights (1.69 GB / world) are far larger
    # than the 126 MB L2 and are streamed once per step, so no separate L2 flush is needed -----------------
    def timed_block(n):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        barrier()
        ev[0].record()
        for _ in range(n):
            step(x, logits)
        ev[1].record()
        barrier()
        t = torch.tensor([ev[0].elapsed_time(ev[1])], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / n

    with ClockSampler(local_rank) as clocks:
        block_ms = [timed_block(args.steps) for _ in range(max(args.blocks, 1))]
    tb.matmul_check_status()
    ms_per_step = median(block_ms)
    value = T * world / (ms_per_step * 1e-3)
    blocks = {"n": len(block_ms), "steps_per_block": args.steps, "ms_per_step_median": ms_per_step,
              "ms_per_step_min": min(block_ms), "ms_per_step_max": max(block_ms)}

    # ---- the dominant kernel: events around the two grouped-GEMM launches of the eager step (every other kernel of the
    # step still runs); a spin kernel ahead of every step lets the host enqueue the step before the GPU reaches it ----
    gt = Spans()
    barrier()
    n_span = min(args.steps, 20)
    for _ in range(n_span):
        torch.cuda._sleep(int(2.0e6 if T > 1024 else 4.0e5))
        eager(x, logits, gt)
    barrier()
    per_step, calls_per_step = gt.per_step_ms(n_span)
    gemm_ms_per_step = median(per_step)
    # routed rows this rank multiplies: read from the routing of its own step, not assumed
    if world == 1:
        col_sum = tb.topk(logits, TOP_K).mask_metadata.col_sum
        rows_local = int(col_sum.sum().item())
        n_active = int((col_sum > 0).sum().item())
    else:
        sp_all = tb.topk(logits, TOP_K, apply_softmax=True, all_gather=True, symm_mem_pool=pool)
        cs = sp_all.mask_metadata.col_sum
        mine = assignment.expt_boolmask[rank].to(cs.device)
        rows_local = int(cs[mine].sum().item())
        n_active = int((cs[mine] > 0).sum().item())
    flop_per_step = rows_local * (FLOP_PER_ROW_FC1 + FLOP_PER_ROW_FC2)
    achieved_tflops = flop_per_step / (gemm_ms_per_step * 1e-3) / 1e12
    per_rank = None
    if world > 1:
        tf = torch.tensor([achieved_tflops, float(rows_local), gemm_ms_per_step], device=dev, dtype=torch.float64)
        allt = [torch.zeros_like(tf) for _ in range(world)]
        dist.all_gather(allt, tf)
        per_rank = [{"rank": r, "tflops": float(t[0]), "rows": int(t[1]), "gemm_ms": float(t[2])} for r, t in enumerate(allt)]
        achieved_tflops = min(p["tflops"] for p in per_rank)            # the slowest rank's

    # ---- one long back-to-back pass: clocks settle where the sustained peak was measured ----------------------
    sustained = None
    if args.sustained_s > 0 and T > 1024:
        n_long = max(int(args.sustained_s * 1e3 / ms_per_step) + 1, args.steps)
        gl = Spans()
        with ClockSampler(local_rank) as lclocks:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            barrier()
            ev[0].record()
            for _ in range(n_long):
                eager(x, logits, gl)
            ev[1].record()
            barrier()
        ms_long = ev[0].elapsed_time(ev[1]) / n_long
        ps, _ = gl.per_step_ms(n_long)
        g_long = median(ps[len(ps) // 2:])                              # second half: clocks have settled
        tf_long = flop_per_step / (g_long * 1e-3) / 1e12
        sustained = {"steps": n_long, "seconds": ms_long * n_long / 1e3, "ms_per_step": ms_long, "gemm_ms_per_step": g_long,
                     "tflops": tf_long, "clocks": lclocks.summary(), "note": "eager steps (no graph), events around the GEMM launches"}

    act_bytes = rows_local * (D_MODEL * 2 + D_FF * 2 * 2 + D_MODEL * 2)
    stream_gbs = (n_active * BYTES_PER_EXPERT + act_bytes) / (gemm_ms_per_step * 1e-3) / 1e9
    decode_kernel = lw.use_block_scaled(T * TOP_K if world == 1 else rows_local)
    roofline = {
        "bound": "tensor",
        "kernel": "gemm_tc_kernel (fc1 + fc2 launches of a step incl. fc1's row gather, bf16 kind::f16 after in-SM dequant)",
        "achieved": achieved_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
        "frac": achieved_tflops / peaks["bf16_tflops"],
        "peak_source": f"{peaks['source']} bf16 cuBLAS, burst (the timed block is short and runs at full clocks)",
        "frac_burst": achieved_tflops / peaks["bf16_tflops"],
        "frac_sustained": None if sustained is None else sustained["tflops"] / peaks["bf16_tflops_sustained"],
        "peak_sustained": peaks["bf16_tflops_sustained"],
        "traffic": gemm_traffic_note(T, N_EXPTS, world),
        "ms_per_step_in_kernel": gemm_ms_per_step, "launches_per_step": calls_per_step,
        "rows_this_rank": rows_local, "per_rank": per_rank,
        "hbm": {"active_experts": n_active, "algorithmic_gbs": stream_gbs, "peak_gbs": peaks["hbm_gbs"],
                "frac": stream_gbs / peaks["hbm_gbs"]},
    }
    if T <= 256 and world == 1:        # decode regime: the grouped GEMM streams weights, HBM is the bound
        if graphed is not None:
            # the eager GEMM spans include launch gaps that the replayed graph does not have: charge the weight bytes
            # to the whole graph step instead (routing and combine included, so this understates the kernel)
            stream_gbs = (n_active * BYTES_PER_EXPERT + act_bytes) / (ms_per_step * 1e-3) / 1e9
            roofline["hbm"].update({"algorithmic_gbs": stream_gbs, "frac": stream_gbs / peaks["hbm_gbs"]})
        roofline.update({"bound": "hbm", "achieved": stream_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": stream_gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
                         "tflops": achieved_tflops, "frac_burst": None, "frac_sustained": None,
                         "kernel": ("gemm_mx_kernel (block-scaled, fc1 + fc2)" if decode_kernel else "gemm_stream_kernel (fc1 + fc2)") +
                                   ", timed as the whole replayed step"})

    # ---- per-phase breakdown of the expert-parallel step (untimed pass, eager) -----------------------------------
    phases = None
    if world > 1:
        names, evs = [], []

        def mark(name):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            names.append(name)
            evs.append(e)

        acc = {}
        n_ph = 5
        for _ in range(n_ph):
            names.clear()
            evs.clear()
            barrier()
            torch.cuda._sleep(int(2.0e6))
            mark("start")
            eager(x, logits, mark=mark)
            torch.cuda.synchronize()
            for i in range(1, len(evs)):
                acc.setdefault(names[i], []).append(evs[i - 1].elapsed_time(evs[i]))
        phases = {k_: median(v) for k_, v in acc.items()}
        phases["note"] = "rank 0, eager step, median of 5; the timed step is the same sequence replayed from a graph"

    # ---- end to end: host buffers in, host result out, through the public API ---------------------------
    e2e = None
    if not args.no_e2e:
        xh = x.cpu().pin_memory()
        lh = logits.cpu().pin_memory()
        zh = [torch.empty((T, D_MODEL), dtype=torch.bfloat16).pin_memory() for _ in range(2)]

        def e2e_block(run, n):
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

        def e2e_time(run, n):                   # median of three K-step blocks, like the device-resident number
            run(3)
            return median([e2e_block(run, n) for _ in range(3)])

        n_e2e = args.steps
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
        h2d, d2h = xh.numel() * 2 + lh.numel() * 4, zh[0].numel() * 2

        # the copies alone, one direction at a time, to name the wall when the end-to-end rate falls short of `value`
        def copy_rate(fn, nbytes):
            fn()
            barrier()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record()
            for _ in range(4):
                fn()
            c1.record()
            barrier()
            return nbytes * 4 / (c0.elapsed_time(c1) * 1e-3) / 1e9

        h2d_gbs = copy_rate(lambda: (xd.copy_(xh, non_blocking=True), ld.copy_(lh, non_blocking=True)), h2d)
        d2h_gbs = copy_rate(lambda: zh[0].copy_(z, non_blocking=True), d2h)
        e2e = {"value": T * world / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "steps": n_e2e, "pipelined": how, "ms_per_step": ms_e2e,
               "achieved_gbs_per_rank": {"h2d_in_step": h2d / (ms_e2e * 1e-3) / 1e9, "d2h_in_step": d2h / (ms_e2e * 1e-3) / 1e9,
                                         "h2d_alone": h2d_gbs, "d2h_alone": d2h_gbs,
                                         "note": "alone = this rank's copies by themselves while every other rank does the same"}}

    # ---- decode on the expert-parallel layer: 64 tokens per rank through the same graphed peer path -----------------
    decode_ep = None
    if want_decode_ep and pool is not None and pool.peer_ok:
        Td = 64
        pool_d = tb.SymmetricMemoryPool(tb.Mesh(dist.group.WORLD))
        pool_d.initialize_matmul(Td * world, D_MODEL, D_MODEL, TOP_K, N_EXPTS, torch.bfloat16, dev)
        if pool_d.enable_peer_buffers(Td, D_MODEL, D_MODEL, TOP_K, torch.bfloat16, dev):
            xd_, ld_ = make_batch(Td, N_EXPTS, dev, 8000 + rank, expert_bias)
            fwd = lambda xi, li: moe_layer_forward_ep(xi, li, lw, TOP_K, assignment, pool_d, exchange=args.exchange)
            gl_ = GraphedMoeLayer(lw, TOP_K, Td, D_MODEL, N_EXPTS, dev, forward=fwd)
            for _ in range(3):
                gl_(xd_, ld_)
            barrier()
            ev3 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev3[0].record()
            nd = 50
            for _ in range(nd):
                gl_(xd_, ld_)
            ev3[1].record()
            barrier()
            td = torch.tensor([ev3[0].elapsed_time(ev3[1]) / nd], device=dev, dtype=torch.float64)
            dist.all_reduce(td, op=dist.ReduceOp.MAX)
            sp_d = tb.topk(ld_, TOP_K, apply_softmax=True, all_gather=True, symm_mem_pool=pool_d)
            csd = sp_d.mask_metadata.col_sum
            act_d = int((csd[assignment.expt_boolmask[rank].to(csd.device)] > 0).sum().item())
            ms_d = float(td.item())
            wb = act_d * BYTES_PER_EXPERT
            decode_ep = {"tokens_per_rank": Td, "ms_per_step": ms_d, "tokens_per_s": Td * world / (ms_d * 1e-3),
                         "active_experts_this_rank": act_d, "weight_gbs_this_rank": wb / ms_d / 1e6,
                         "frac_hbm": wb / ms_d / 1e6 / peaks["hbm_gbs"],
                         "note": "whole expert-parallel step replayed from a CUDA graph (routing, peer exchange, fc1, fc2, "
                                 "combine); the same batch every step: a rank's active experts (up to 211 MB) exceed L2"}
        barrier()

    sub = {}
    if want_sub and rank == 0:
        sub["decode"] = decode_record(lw, dev, expert_bias, peaks)
        sub["sweep_20b"] = sweep_20b_record(slice_experts(lw, 32), dev, expert_bias, peaks)
        sub["micro"] = micro_record(dev, peaks)
        sub["tensor_roofs"] = tensor_roof_record(dev)
        sub["act_fp8"] = act_fp8_record(lw, dev, expert_bias, peaks, T, 10, sub["tensor_roofs"])
        sub["act_fp8"]["gemm_speedup_vs_bf16_path"] = sub["act_fp8"]["gemm_tflops"] / achieved_tflops
        roofline["tensor_pipe_roofs_measured"] = sub["tensor_roofs"]["tflops"]

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_baseline_record(3, full=True)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(T, world),
                       "cuda_graph": graphed is not None,
                       "expert_placement": placement_note,
                       "exchange": None if world == 1 else ("peer-mapped buffers" if pool.peer_ok else
                                                            f"NCCL all-to-all ({pool.peer_error})"),
                       "ep_overlap": None if world == 1 else {"chunks": args.ep_chunks, "idle_sms": args.ep_idle_sms},
                       "l2": "inputs larger than L2 (weights streamed once per step)",
                       "tflops_per_step_algorithmic": T * world * TOP_K * (FLOP_PER_ROW_FC1 + FLOP_PER_ROW_FC2) / 1e12},
            "clocks": clocks.summary(), "blocks": blocks, "sustained": sustained, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_note": f"{launches_per_step} kernels of this library per step, counted by the library at its launch sites",
            "parity": parity, "roofline": roofline, "phases_ms": phases, "decode_ep": decode_ep, "cpu_baseline": cpu_baseline,
        }
        line.update(sub)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
