"""Generate the golden fixtures in this folder by running the REFERENCE's own torch
implementations on the CPU.

Usage (only where the reference checkout is available; the fixtures are committed):

    python tests/golden/make_golden.py /path/to/reference

The reference package (``python/triton_kernels``) is imported unmodified.  Shims applied
by this script, none of which touches the arithmetic that is recorded:

* ``triton.language.target_info.is_hip_gfx1250`` is added when the installed triton lacks it
  (import-time only);
* ``torch.histc`` on int32 CPU tensors is served by ``torch.bincount`` (same histogram);
* ``SparseMatrix`` inside ``topk_torch`` is replaced by a plain record, because its
  ``__post_init__`` launches GPU kernels;
* inside ``matmul_torch`` the GPU dequantiser is replaced by the reference's own
  ``upcast_from_mxfp_torch`` and a hard-coded ``device="cuda"`` of an index helper is dropped.

Every fixture is an ``.npz``; bf16/fp16 arrays are stored as their uint16 bit patterns
(key suffix ``__bf16`` / ``__fp16``).
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def pack(d):
    out = {}
    for k, v in d.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().contiguous()
            if v.dtype == torch.bfloat16:
                out[k + "__bf16"] = v.view(torch.uint16).numpy()
            elif v.dtype == torch.float16:
                out[k + "__fp16"] = v.view(torch.uint16).numpy()
            elif v.dtype == torch.uint32:
                out[k] = v.view(torch.int32).numpy()
            else:
                out[k] = v.numpy()
        else:
            out[k] = np.asarray(v)
    return out


def save(name, d):
    np.savez_compressed(HERE / f"{name}.npz", **pack(d))
    print("wrote", name, {k: tuple(np.asarray(v).shape) for k, v in pack(d).items()})


def main(ref_root):
    sys.path.insert(0, str(Path(ref_root) / "python" / "triton_kernels"))
    import triton.language.target_info as ti
    if not hasattr(ti, "is_hip_gfx1250"):
        ti.is_hip_gfx1250 = lambda: False
    import triton_kernels.topk as ref_topk
    import triton_kernels.matmul as ref_matmul
    import triton_kernels.numerics_details.mxfp as ref_mxfp
    from triton_kernels.numerics_details.mxfp import (DequantScaleRoundingMode, downcast_to_mxfp_torch,
                                                      upcast_from_mxfp_torch)
    from triton_kernels.tensor_details.bitmatrix import make_bitmatrix_metadata_torch
    from triton_kernels.tensor_details.ragged_tensor import (make_ragged_tensor_metadata_torch,
                                                             remap_ragged_tensor_metadata_torch)
    from triton_kernels.swiglu import swiglu_torch, PrecisionConfig as SwigluPC
    from triton_kernels.reduce import reduce_torch
    from triton_kernels.tensor import wrap_torch_tensor
    from triton_kernels.tensor_details.dtype import FP4
    from triton_kernels.tensor_details.layout_details.blackwell_scale import BlackwellMXScaleLayout
    from triton_kernels.tensor_details.layout_details.blackwell_value import BlackwellMXValueLayout

    # ---- shims ------------------------------------------------------------------------------
    real_histc = torch.histc

    def histc(x, bins, min=0, max=0):
        if x.dtype in (torch.int32, torch.int64):
            x = x[(x >= 0) & (x <= max)]
            return torch.bincount(x.long(), minlength=bins)[:bins].float()
        return real_histc(x, bins=bins, min=min, max=max)

    torch.histc = histc
    ref_topk.SparseMatrix = lambda vals, indx, mask: types.SimpleNamespace(vals=vals, indx=indx, mask=mask)
    ref_mxfp.upcast_from_mxfp = lambda t, s, dt, axis, tensor_scale=None: upcast_from_mxfp_torch(t, s, dt, axis)
    real_arange = torch.arange

    def arange(*a, **kw):
        kw.pop("device", None)
        return real_arange(*a, **kw)

    # ---- quantiser ----------------------------------------------------------------------------
    g = torch.Generator().manual_seed(0)
    cases = [
        ("mxfp_bf16_last", (37, 256), -1, torch.bfloat16, DequantScaleRoundingMode.ROUND_UP),
        ("mxfp_bf16_axis1", (3, 128, 40), 1, torch.bfloat16, DequantScaleRoundingMode.ROUND_UP),
        ("mxfp_fp16_axis0_down", (32, 30, 12), 0, torch.float16, DequantScaleRoundingMode.ROUND_DOWN),
        ("mxfp_fp32_last", (5, 7, 96), 2, torch.float32, DequantScaleRoundingMode.ROUND_UP),
        ("mxfp_bf16_outliers", (64, 512), 1, torch.bfloat16, DequantScaleRoundingMode.ROUND_UP),
    ]
    for name, shape, axis, dt, mode in cases:
        x = torch.randn(shape, generator=g)
        if "outliers" in name:
            x = torch.where(torch.rand(shape, generator=g) < 0.01, x * 100, x)
        # spread magnitudes so that scales and subnormal e2m1 codes are exercised
        x = (x * torch.exp2(torch.randint(-12, 12, shape[:1] + (1,) * (len(shape) - 1), generator=g).float())).to(dt)
        q, s = downcast_to_mxfp_torch(x, torch.uint8, axis, DEQUANT_SCALE_ROUNDING_MODE=mode)
        d = {"x": x, "q": q.contiguous(), "scale": s.contiguous(), "axis": axis, "mode": mode.value}
        for tname, tdt in (("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)):
            d["deq_" + tname] = upcast_from_mxfp_torch(q, s, tdt, axis).contiguous()
        save(name, d)

    # ---- top-k + bitmatrix metadata ---------------------------------------------------------------
    for T, E, k, sm in [(7, 13, 4, True), (256, 128, 4, True), (300, 200, 8, False), (33, 32, 2, True)]:
        logits = torch.randn(T, E, generator=g)
        logits[:, 1] = logits[:, 0]                      # exact ties -> smaller index wins
        sp = ref_topk.topk_torch(logits, k, apply_softmax=sm)
        meta = make_bitmatrix_metadata_torch(sp.indx, sp.mask)
        save(f"topk_T{T}_E{E}_k{k}", {
            "logits": logits, "k": k, "softmax": int(sm), "vals": sp.vals, "indx": sp.indx,
            "bitmatrix": sp.mask.storage.data.contiguous(), "col_sum": meta.col_sum,
            "col_sorted": meta.col_sorted_indx.int(), "row_sorted": meta.row_sorted_indx.int()})

    # ---- ragged metadata + remap ---------------------------------------------------------------------
    for n_slices in (1, 7, 33, 130):
        sizes = torch.randint(0, 200, (n_slices,), generator=g, dtype=torch.int32)
        sizes[n_slices // 2] = 0
        n_rows = int(sizes.sum()) + 17
        m = make_ragged_tensor_metadata_torch(sizes, n_rows)
        smap = torch.full((n_slices,), -1, dtype=torch.int32)
        keep = torch.randperm(n_slices, generator=g)[: max(1, n_slices - 3)].sort().values
        smap[keep] = torch.arange(keep.numel(), dtype=torch.int32)
        r = remap_ragged_tensor_metadata_torch(m, smap)
        save(f"ragged_E{n_slices}", {
            "slice_sizes": sizes, "n_rows": n_rows, "slice_offs": m.slice_offs, "block_offs": m.block_offs_data,
            "block_schedule": m.block_schedule_data, "slice_map": smap, "r_slice_sizes": r.slice_sizes,
            "r_slice_offs": r.slice_offs, "r_block_offs": r.block_offs_data,
            "r_block_schedule": r.block_schedule_data})

    # ---- ragged GEMM (bf16 x MXFP4), SwiGLU, combine -------------------------------------------------
    E, K, N, M, k = 4, 96, 64, 50, 2
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(E, K, N, generator=g) * 0.1).bfloat16()
    wq, ws = downcast_to_mxfp_torch(w, torch.uint8, axis=1)
    bias = torch.randn(E, N, generator=g)
    sizes = torch.tensor([13, 0, 29, 8], dtype=torch.int32)
    n_rows = int(sizes.sum())
    gather = torch.randint(0, M, (n_rows,), generator=g, dtype=torch.int32)
    scatter = torch.randperm(n_rows, generator=g).int()
    gammas = torch.rand(n_rows, generator=g)
    meta = make_ragged_tensor_metadata_torch(sizes, n_rows)
    pc = ref_matmul.PrecisionConfig(b_mx_scale=wrap_torch_tensor(ws), b_microblock_size=32)
    torch.arange = arange
    try:
        y = ref_matmul.matmul_torch(x, wrap_torch_tensor(wq, dtype=FP4), bias, meta, None, gather, scatter, pc,
                                    gammas=gammas)
        y_plain = ref_matmul.matmul_torch(x[:n_rows].contiguous(), wrap_torch_tensor(wq, dtype=FP4), bias, meta, None,
                                          None, None, pc)
    finally:
        torch.arange = real_arange
    act = swiglu_torch(y_plain, 1.702, SwigluPC(limit=7.0))
    yk = torch.randn(25, k, 48, generator=g).bfloat16()
    mask = (torch.rand(25, k, 1, generator=g) > 0.3).expand(25, k, 48)
    red, _ = reduce_torch(yk, 1, mask=mask, x_flex=None, y_flex=None)
    red_scaled, _ = reduce_torch(yk, 1, scale=torch.rand(25, k, 1, generator=g), x_flex=None, y_flex=None)
    save("gemm_small", {
        "x": x, "wq": wq.contiguous(), "ws": ws.contiguous(), "bias": bias, "slice_sizes": sizes, "gather": gather,
        "scatter": scatter, "gammas": gammas, "y": y, "y_plain": y_plain, "act": act, "alpha": 1.702, "limit": 7.0,
        "yk": yk, "mask": mask.contiguous(), "red": red})
    _ = red_scaled

    # ---- Blackwell weight layouts -------------------------------------------------------------------------
    s = torch.randint(0, 255, (3, 10, 200), generator=g, dtype=torch.uint8)
    sw = BlackwellMXScaleLayout().make_transformation([3, 10, 200], False).swizzle_data(s)
    v = torch.randint(0, 255, (2, 96, 20), generator=g, dtype=torch.uint8)      # canonical: [E, K, N/2]
    tv = BlackwellMXValueLayout().make_transformation([2, 96, 40], True)
    vw = tv.swizzle_data(v)
    save("layout_bw", {"scale": s, "scale_swizzled": sw.contiguous(), "value": v,
                       "value_swizzled": vw.contiguous(), "value_swizzled_strides": list(vw.stride())})
    # the pre-tiled value layout and the activation scale layout (their torch paths; the ragged activation form pads
    # with a GPU kernel in the reference and is not recorded)
    from triton_kernels.tensor_details.layout_details.blackwell_value_shuffled import BlackwellMX4ValueShuffledLayout
    from triton_kernels.tensor_details.layout_details.blackwell_scale import BlackwellActMXScaleLayout
    v2 = torch.randint(0, 255, (2, 200, 150), generator=g, dtype=torch.uint8)    # canonical [E, K, N/2]: K = 200, N = 300
    tsh = BlackwellMX4ValueShuffledLayout(block_k=128, block_n=256).make_transformation([2, 200, 300], True)
    vs = tsh.swizzle_data(v2)
    tsh2 = BlackwellMX4ValueShuffledLayout(block_k=64, block_n=128).make_transformation([2, 200, 300], True)
    vs2 = tsh2.swizzle_data(v2)
    a = torch.randint(0, 255, (300, 10), generator=g, dtype=torch.uint8)          # activation scales [M, K/32]
    ta = BlackwellActMXScaleLayout(None).make_transformation([300, 10], False)
    asw = ta.swizzle_data(a)
    save("layout_bw2", {"value": v2, "value_shuffled_128_256": vs.contiguous(), "value_shuffled_64_128": vs2.contiguous(),
                        "act_scale": a, "act_scale_swizzled": asw.contiguous()})
    # ---- router: dense product + top-k (bench/bench_mlp.py:70 followed by topk) -------------------------------------
    for T, K, E, k in [(50, 96, 32, 4), (9, 64, 128, 2)]:
        x = torch.randn(T, K, generator=g).bfloat16()
        wg = (torch.randn(K, E, generator=g) / K ** 0.5).bfloat16()
        bg = torch.randn(E, generator=g)
        torch.arange = arange
        try:
            logits = ref_matmul.matmul_torch(x, wg, bg, None, None, None, None, ref_matmul.PrecisionConfig())
        finally:
            torch.arange = real_arange
        sp = ref_topk.topk_torch(logits, k, apply_softmax=True)
        save(f"router_T{T}_E{E}_k{k}", {"x": x, "wg": wg, "bg": bg, "k": k, "logits": logits, "vals": sp.vals, "indx": sp.indx,
                                         "bitmatrix": sp.mask.storage.data.contiguous()})
    torch.histc = real_histc


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a triton-lang/triton checkout>")
    main(sys.argv[1])
