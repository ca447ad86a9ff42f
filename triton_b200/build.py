"""Build libmoe_b200.so (all CUDA kernels + the C ABI) for sm_100a with nvcc.

    python -m triton_b200.build            # incremental: rebuilds when a source is newer than the library
    python -m triton_b200.build --force

The library is written next to this file so that it travels with the source tree.
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libmoe_b200.so"
SOURCES = ["api.cu", "mxfp.cu", "routing.cu", "elementwise.cu", "layout.cu", "gemm.cu", "gemm_simt.cu",
           "gemm_tcgen05.cu", "gemm_tcgen05_pair.cu", "gemm_stream.cu", "gemm_mx.cu", "tensor_roof.cu", "router.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libmoe_b200.so cannot be built")


def sources():
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def needs_build():
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "moe_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs, procs = [], []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src.name}\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {src.name}\n{out}\n")
    if failed:
        raise RuntimeError("libmoe_b200.so: compilation failed")
    tmp = LIB.with_suffix(".so.tmp")
    subprocess.check_call([nvcc, "-shared", "-o", str(tmp), *objs, "-Xcompiler", "-fPIC"])
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
