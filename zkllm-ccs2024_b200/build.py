"""Builds libzkllm_b200.so (sm_100a only) from csrc/ with nvcc.

    python zkllm-ccs2024_b200/build.py [--force] [--verbose-ptxas]

Objects go to zkllm-ccs2024_b200/build/, the library to
zkllm-ccs2024_b200/lib/libzkllm_b200.so.  A translation unit is recompiled only
when it or one of the headers is newer than its object.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "lib" / "libzkllm_b200.so"
SOURCES = ["common.cu", "fr_ops.cu", "sumcheck.cu", "g1_ops.cu", "msm.cu", "nn_ops.cu", "bench_kernels.cu", "hostapi.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _headers_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.hpp")) + [HERE.parent / "include" / "zkllm_b200.h"]
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = BUILD / (src + ".o")
    srcp = CSRC / src
    if not force and obj.exists() and obj.stat().st_mtime > max(srcp.stat().st_mtime, _headers_mtime()):
        return f"up to date: {src}"
    cmd = ["nvcc", *NVCC_FLAGS, "-c", str(srcp), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return f"compiled: {src}" + (("\n" + res.stderr) if verbose else "")


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    srcs = [s for s in SOURCES if (CSRC / s).exists()]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for msg in ex.map(lambda s: _compile(s, force, verbose), srcs):
            print(msg)
    objs = [str(BUILD / (s + ".o")) for s in srcs]
    newest = max(Path(o).stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs, "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        print(f"linked: {LIB}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose-ptxas" in sys.argv)
