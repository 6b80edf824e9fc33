"""Builds the CUDA library in-tree: ``zllm_b200/lib/libzq_b200.so`` (sm_100a only, nvcc)."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(OUT_DIR, "libzq_b200.so")
SOURCES = ["zq_api.cu", "zq_codec.cu", "zq_norm.cu", "zq_rope.cu", "zq_gemv.cu", "zq_gemv_resident.cu", "zq_gemv_i8.cu", "zq_gemv_wl.cu", "zq_dist.cu", "zq_qmv.cu", "zq_gemm.cu", "zq_moe.cu", "zq_moe_grouped.cu", "zq_moe_ep.cu", "zq_gguf.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--cudart", "static", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "zq_b200.h"))
    objects = [os.path.join(OUT_DIR, src.replace(".cu", ".o")) for src in SOURCES]
    logs = []

    def compile_one(src: str):
        path = os.path.join(CSRC, src)
        obj = os.path.join(OUT_DIR, src.replace(".cu", ".o"))
        if not (force or _stale(obj, [path] + headers)):
            return src, 0, ""
        r = subprocess.run([_nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj], capture_output=True, text=True)
        return src, r.returncode, r.stdout + r.stderr

    # the translation units are independent: compile them side by side
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as pool:
        for src, code, log in pool.map(compile_one, SOURCES):
            logs.append(log)
            if code != 0:
                sys.stderr.write(log)
                raise RuntimeError(f"nvcc failed on {src}")
    if force or _stale(LIB, objects):
        r = subprocess.run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "--cudart", "static", "-o", LIB, *objects, "-lpthread", "-ldl"], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    if verbose:
        sys.stderr.write("".join(logs))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
