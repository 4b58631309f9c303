"""Build liblhb200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m longhornai_b200.build [--force] [--verbose]

The library has no dependency on PyTorch or on libcuda at link time (the CUDA
runtime is linked statically; the one driver entry point it needs is resolved
at run time), so it also loads on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "_obj")
LIB = os.path.join(PKG, "lib", "liblhb200.so")

SOURCES = ["api.cu", "quant.cu", "gemm_generic.cu", "kvcache.cu", "paged_attention_generic.cu",
           "tensor_map.cu", "gemv_mma.cu", "gemm_w4a16_tc.cu", "gemm_w8a8_tc.cu", "paged_attention_decode.cu",
           "cache_manager.cu", "glue.cu", "quant_asym.cu", "fp8.cu", "peer_gather.cu", "peer_vmm.cu", "lh_dropin.cu"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
              "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]
# extra compiler flags for development builds, e.g. LHB_NVCC_EXTRA="-DLHB_GEMV_TRACE"
NVCC_FLAGS += os.environ.get("LHB_NVCC_EXTRA", "").split()


def _deps_mtime():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".hpp"))]
    hdrs += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))
             if f.endswith((".h", ".hpp"))]
    inc_lh = os.path.join(ROOT, "include", "lh")
    if os.path.isdir(inc_lh):
        for dp, _, fs in os.walk(inc_lh):
            hdrs += [os.path.join(dp, f) for f in fs]
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, verbose):
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    hdr_t = _deps_mtime()
    todo = []
    for s in srcs:
        obj = os.path.join(OBJ, s.replace(".cu", ".o"))
        src_t = max(os.path.getmtime(os.path.join(CSRC, s)), hdr_t)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < src_t:
            todo.append(s)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for src, rc, out in ex.map(lambda s: _compile(s, verbose), todo):
                if verbose or rc != 0:
                    print(f"--- {src}\n{out}", file=sys.stderr)
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {src}")
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in srcs]
    if todo or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = ["nvcc", "-shared", "-cudart", "static", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            print(r.stdout + r.stderr, file=sys.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
