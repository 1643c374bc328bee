"""ctypes access to oracle/_build/libzkoracle.so (TEST INFRASTRUCTURE ONLY).

Used by tests/ at sizes where the Python big-integer oracle is too slow and by
bench.py for the timed CPU baseline.  Never imported by the product package."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "_build" / "libzkoracle.so"
_lib = None


def build() -> Path:
    subprocess.run(["make", "-C", str(_HERE), "cpu"], check=True, capture_output=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        if not _LIB.exists():
            build()
        _lib = ctypes.CDLL(str(_LIB))
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


sz = ctypes.c_size_t


def threads() -> int:
    return int(lib().zko_threads())


def fr_mul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    out = np.empty_like(a)
    lib().zko_fr_mul(_p(a), _p(b), _p(out), sz(a.shape[0]))
    return out


def fr_inv(a: np.ndarray) -> np.ndarray:
    out = np.empty_like(a)
    lib().zko_fr_inv(_p(a), _p(out), sz(a.shape[0]))
    return out


def g1_add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    out = np.empty_like(a)
    lib().zko_g1_add(_p(a), _p(b), _p(out), sz(a.shape[0]))
    return out


def g1_normalise(a: np.ndarray) -> np.ndarray:
    """Jacobian -> (x, y, 1) representative (all zero for the identity), for equality tests"""
    a = np.ascontiguousarray(a, dtype=np.uint32).reshape(-1, 36)
    out = np.empty_like(a)
    lib().zko_g1_to_affine_jac(_p(a), _p(out), sz(a.shape[0]))
    return out


def g1_mul(g: np.ndarray, k: np.ndarray) -> np.ndarray:
    out = np.empty_like(g)
    lib().zko_g1_mul(_p(g), _p(k), _p(out), sz(g.shape[0]))
    return out


def commit_int(gens: np.ndarray, scalars: np.ndarray, algo: str = "pippenger", nthreads: int = 0) -> np.ndarray:
    gens = np.ascontiguousarray(gens, dtype=np.uint32).reshape(-1, 36)
    scalars = np.ascontiguousarray(scalars, dtype=np.int32)
    n = gens.shape[0]
    m = scalars.size // n
    out = np.empty((m, 36), dtype=np.uint32)
    fn = lib().zko_commit_int_pippenger if algo == "pippenger" else lib().zko_commit_int_ref
    fn(_p(gens), sz(n), _p(scalars), sz(m), _p(out), ctypes.c_int(nthreads))
    return out


def mle_eval(a: np.ndarray, u: np.ndarray) -> np.ndarray:
    out = np.empty((1, 8), dtype=np.uint32)
    u = np.ascontiguousarray(u, dtype=np.uint32).reshape(-1, 8)
    uu = u if u.shape[0] else np.zeros((1, 8), dtype=np.uint32)
    lib().zko_mle_eval(_p(a), sz(a.shape[0]), _p(uu), ctypes.c_uint(u.shape[0]), _p(out))
    return out


def zkfc_prove(X, W, Y, B, I, O, ub, ui, uo):
    kI = ui.shape[0]
    polys = np.zeros((max(3 * kI, 1), 8), dtype=np.uint32)
    claims = np.zeros((4, 8), dtype=np.uint32)
    pad = lambda u: u if u.shape[0] else np.zeros((1, 8), dtype=np.uint32)
    rc = lib().zko_zkfc_prove(_p(X), _p(W), _p(Y), sz(B), sz(I), sz(O), _p(pad(ub)), _p(pad(ui)), _p(pad(uo)), _p(polys), _p(claims))
    return rc, polys[:3 * kI], claims


def tlookup_prove(S, T, m, alpha, beta, u, v, nthreads: int = 0):
    D, N = S.shape[0], T.shape[0]
    kD = u.shape[0]
    polys = np.zeros((max(4 * kD, 1), 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    pad = lambda x: x if x.shape[0] else np.zeros((1, 8), dtype=np.uint32)
    rc = lib().zko_tlookup_prove(_p(S), _p(T), _p(m), sz(D), sz(N), _p(alpha), _p(beta), _p(pad(u)), _p(pad(v)),
                                 _p(polys), _p(final), ctypes.c_int(nthreads))
    return rc, polys[:4 * kD], final


def me_open(t: np.ndarray, gens: np.ndarray, u: np.ndarray):
    """Commitment::me_open: returns (proof [3k+1, 36] Jacobian points, final scalar [1, 8])."""
    n, k = t.shape[0], u.shape[0]
    proof = np.zeros((3 * k + 1, 36), dtype=np.uint32)
    out = np.zeros((1, 8), dtype=np.uint32)
    pad = u if k else np.zeros((1, 8), dtype=np.uint32)
    lib().zko_me_open(_p(t), _p(gens), sz(n), _p(pad), ctypes.c_uint(k), _p(proof), _p(out))
    return proof, out
