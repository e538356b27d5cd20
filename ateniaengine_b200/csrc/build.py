"""Builds libatenia_moe.so (sm_100a only) with nvcc.  Used by __graft_entry__.build()."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["grouped_gemm.cu", "w8_gemm.cu", "w8_gemm_m256.cu", "bf16_decode_gemm.cu", "decode_gemv.cu", "grouped_gemm_2cta.cu", "router.cu", "router_dmma.cu", "router_splitk.cu", "dispatch.cu", "combine.cu", "moe_layer.cu", "ep.cu", "registry.cu", "noalloc.cu", "planner.cu", "stack.cu", "tier.cu", "dense_int8.cu"]
LIB = os.path.join(HERE, "libatenia_moe.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-ccbin", "g++",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v"]


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    headers = [os.path.join(HERE, h) for h in ("common.cuh", "layer.cuh", "tc_common.cuh", "v3_route.cuh", "route_warp.cuh")] + [
        os.path.join(HERE, "..", "..", "include", "atenia_moe.h")]
    objs = []
    jobs = []
    for src in SOURCES:
        s = os.path.join(HERE, src)
        o = os.path.join(HERE, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append([NVCC] + FLAGS + ["-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        return r.stderr

    with ThreadPoolExecutor(max_workers=8) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        for l in logs:
            sys.stderr.write(l)
    if jobs or force or _stale(LIB, objs):
        run([NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++",
                                                    "-lnccl"])
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
