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
SOURCES = ["common.cu", "fr_ops.cu", "sumcheck.cu", "combine.cu", "g1_ops.cu", "msm.cu", "nn_ops.cu", "bench_kernels.cu", "comm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _deps_mtime(path: Path, seen=None) -> float:
    """newest modification time among a source file and the local headers it includes, directly or not"""
    import re
    seen = set() if seen is None else seen
    if path in seen or not path.exists():
        return 0.0
    seen.add(path)
    newest = path.stat().st_mtime
    for inc in re.findall(r'^\s*#\s*include\s+"([^"]+)"', path.read_text(), flags=re.M):
        newest = max(newest, _deps_mtime((path.parent / inc).resolve(), seen))
    return newest


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = BUILD / (src + ".o")
    srcp = CSRC / src
    if not force and obj.exists() and obj.stat().st_mtime > _deps_mtime(srcp):
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
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs, "-lcudart", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        print(f"linked: {LIB}")
    return LIB


HOST = HERE / "host"
HOST_SOURCES = ["ioutils", "fr-tensor", "polynomial", "g1-tensor", "commitment", "proof", "zkfc", "tlookup", "rescaling", "zksoftmax", "zkrelu"]
HOST_LIB = HERE / "lib" / "libzkllm_host.so"
BIN = HERE / "bin"
STAGES = ["ppgen", "commit-param", "rmsnorm", "self-attn", "ffn", "skip-connection"]
HOST_CXX = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{' '.join(map(str, cmd))} failed:\n{res.stdout}\n{res.stderr}")


def build_host(force: bool = False) -> Path:
    """The C++ classes with the reference's names (host/), as libzkllm_host.so, and
    the stage driver bin/zkllm-driver with one symlink per stage name."""
    out = BUILD / "host"
    out.mkdir(parents=True, exist_ok=True)
    BIN.mkdir(exist_ok=True)
    newest_hdr = max(p.stat().st_mtime for p in list(HOST.glob("*.cuh")) + list(HOST.glob("*.hpp")) + [CSRC / "hostfr.hpp"])

    def one(name):
        src, obj = HOST / f"{name}.cpp", out / f"{name}.o"
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_hdr):
            _run([HOST_CXX, "-std=c++17", "-O2", "-fPIC", "-Wall", "-c", str(src), "-o", str(obj)])
        return str(obj)

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(one, HOST_SOURCES))
        drv = one("drivers")
    _run([HOST_CXX, "-shared", "-o", str(HOST_LIB), *objs, f"-L{LIB.parent}", "-lzkllm_b200", "-Wl,-rpath,$ORIGIN"])
    exe = BIN / "zkllm-driver"
    _run([HOST_CXX, "-o", str(exe), drv, f"-L{LIB.parent}", "-lzkllm_host", "-lzkllm_b200", "-Wl,-rpath,$ORIGIN/../lib"])
    for st in STAGES:
        link = BIN / st
        if link.is_symlink() or link.exists():
            link.unlink()
        link.symlink_to("zkllm-driver")
    print(f"linked: {HOST_LIB} and {exe}")
    return HOST_LIB


def reference_dir():
    """Where the reference's sources are, or None: $ZKLLM_REFERENCE_DIR, else a directory named `reference` next to
    this repository.  Only the drop-in check (build_reference_drivers) and the test checkers use it."""
    cands = []
    if os.environ.get("ZKLLM_REFERENCE_DIR"):
        cands.append(Path(os.environ["ZKLLM_REFERENCE_DIR"]))
    cands.append(HERE.parent.parent / "reference")
    for c in cands:
        if (c / "commitment.cu").exists():
            return c
    return None


def build_reference_drivers(ref_dir: Path) -> bool:
    """Drop-in check: the reference's six driver sources, unmodified, compiled against
    host/ and linked with the two libraries, into bin/ref-drivers/.  Each source is
    compiled from a scratch copy, because a quoted #include looks beside the
    including file first and would find the reference's own headers there."""
    import shutil
    import tempfile
    if not all((ref_dir / f"{st}.cu").exists() for st in STAGES):
        return False
    dst = BIN / "ref-drivers"
    dst.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        for st in STAGES:
            shutil.copy(ref_dir / f"{st}.cu", Path(tmp) / f"{st}.cu")
            obj = Path(tmp) / f"{st}.o"
            _run([HOST_CXX, "-x", "c++", "-std=c++17", "-O1", f"-I{HOST}", "-c", str(Path(tmp) / f"{st}.cu"), "-o", str(obj)])
            _run([HOST_CXX, "-o", str(dst / st), str(obj), f"-L{LIB.parent}", "-lzkllm_host", "-lzkllm_b200",
                  "-Wl,-rpath,$ORIGIN/../../lib"])
    print(f"reference drivers built unmodified against host/: {dst}")
    return True


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose-ptxas" in sys.argv)
    build_host(force="--force" in sys.argv)
    if reference_dir() is not None:
        build_reference_drivers(reference_dir())
