"""ctypes binding of libzkllm_b200.so, the B200 prover core.

The library is the product; this module only loads it and gives tests, the
benchmark and the smoke test a thin way to call its C ABI (include/zkllm_b200.h)
with numpy arrays.  There is no CPU fallback: if the shared library is missing,
or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
# ZKLLM_B200_LIB selects another build of the same library (e.g. a tuning variant)
LIB_PATH = Path(os.environ["ZKLLM_B200_LIB"]) if os.environ.get("ZKLLM_B200_LIB") else _HERE / "lib" / "libzkllm_b200.so"

OK, ERR_CUDA, ERR_DIM, ERR_VERIFY, ERR_ARG, ERR_LIMIT = 0, -1, -2, -3, -4, -5


class ZkbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the shared library once; fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(
                f"{LIB_PATH} not found: build it with `python zkllm-ccs2024_b200/build.py` "
                "(there is no CPU fallback)")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.zkb_last_error.restype = ctypes.c_char_p
        _lib.zkb_launch_count.restype = ctypes.c_ulonglong
    return _lib


def exported_symbols_from_header() -> list:
    """Names of every function declared in include/zkllm_b200.h."""
    import re
    text = (_HERE.parent / "include" / "zkllm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zkb_[a-z0-9_]+)\s*\(", text)))


def _p(x):
    """ctypes argument for: device pointer (int), numpy array (host), None."""
    if x is None:
        return ctypes.c_void_p(0)
    if isinstance(x, DeviceBuffer):
        c = ctypes.c_void_p(x.ptr)
        c._keep = x          # the buffer must outlive the call even when passed as a temporary
        return c
    if isinstance(x, np.ndarray):
        assert x.flags["C_CONTIGUOUS"]
        c = x.ctypes.data_as(ctypes.c_void_p)
        c._keep = x
        return c
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    raise TypeError(type(x))


def call(name: str, *args):
    """Calls a zkb_* entry point; raises ZkbError on a non-zero status."""
    fn = getattr(lib(), name)
    rc = fn(*args)
    if rc != 0:
        raise ZkbError(rc, lib().zkb_last_error().decode())
    return rc


def launch_count() -> int:
    return int(lib().zkb_launch_count())


sz = ctypes.c_size_t
u32 = ctypes.c_uint
u64 = ctypes.c_uint64
i32 = ctypes.c_int32
f64 = ctypes.c_double


class DeviceBuffer:
    """Owns a device allocation made through zkb_malloc."""

    def __init__(self, nbytes: int):
        p = ctypes.c_void_p()
        call("zkb_malloc", ctypes.byref(p), sz(max(int(nbytes), 16)))
        self.ptr = p.value
        self.nbytes = int(nbytes)

    @classmethod
    def from_host(cls, arr: np.ndarray, stream: int = 0) -> "DeviceBuffer":
        arr = np.ascontiguousarray(arr)
        buf = cls(arr.nbytes)
        if arr.nbytes:
            call("zkb_memcpy_h2d", _p(buf), _p(arr), sz(arr.nbytes), _p(stream))
        return buf

    def to_host(self, dtype, shape, stream: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= max(self.nbytes, 16)
        if out.nbytes:
            call("zkb_memcpy_d2h", _p(out), _p(self), sz(out.nbytes), _p(stream))
        return out

    def free(self):
        if self.ptr:
            call("zkb_free", _p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def fr_buffer(limbs: np.ndarray) -> DeviceBuffer:
    """(n, 8) uint32 host array -> device Fr tensor"""
    limbs = np.ascontiguousarray(limbs, dtype=np.uint32).reshape(-1, 8)
    return DeviceBuffer.from_host(limbs)


def fr_host(vals_limbs) -> np.ndarray:
    """contiguous (k, 8) uint32 host array for challenge vectors (k may be 0)"""
    a = np.ascontiguousarray(vals_limbs, dtype=np.uint32).reshape(-1, 8)
    if a.shape[0] == 0:
        a = np.zeros((1, 8), dtype=np.uint32)   # a valid pointer for empty vectors
    return a
