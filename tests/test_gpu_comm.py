"""The library's own communicator (NCCL, csrc/comm.cu) and the sharded provers built on it.

On one GPU the communicator has a single rank: every sharded entry point must then return exactly
what its single-GPU counterpart returns (the exchange is a gather of one block).  With two or more
GPUs visible, two processes (one per GPU) prove the same inputs split between them and every rank
must again return the single-GPU result; that case is skipped on a one-GPU box.  The host-side
combination logic for 2 ranks is also covered on CPU by tests/test_sharding_gloo.py and, with every
rank's share going through the real kernels in one process, by tests/test_gpu_large.py."""
import ctypes
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

from oracle import pyref as R
from tests.util import Dev

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def dev(zkb):
    # PyTorch brings its own NCCL; a process that uses both loads PyTorch's first, and the library then shares that copy
    import torch  # noqa: F401
    d = Dev(zkb)
    rank, world = ctypes.c_int(-1), ctypes.c_int(-1)
    zkb.call("zkb_comm_info", ctypes.byref(rank), ctypes.byref(world))
    if world.value == 0:
        ident = np.zeros(128, dtype=np.uint8)
        zkb.call("zkb_comm_unique_id", zkb._p(ident))
        zkb.call("zkb_comm_init", ctypes.c_int(0), ctypes.c_int(1), zkb._p(ident))
    yield d
    zkb.call("zkb_comm_destroy")


def _rand_fr(rng, k):
    v = rng.integers(0, 1 << 32, size=(max(k, 1), 8), dtype=np.uint64).astype(np.uint32)
    v[:, 7] %= np.uint32(R.R_MOD >> 224)
    return v[:k] if k else np.zeros((1, 8), dtype=np.uint32)


def _ints_to_limbs(v):
    return R.fr_pack([R.int_to_fr(int(x)) for x in np.asarray(v).reshape(-1)])


def test_comm_info_and_double_init(dev):
    z = dev.z
    rank, world = ctypes.c_int(-1), ctypes.c_int(-1)
    z.call("zkb_comm_info", ctypes.byref(rank), ctypes.byref(world))
    assert (rank.value, world.value) == (0, 1)
    with pytest.raises(z.ZkbError) as e:
        z.call("zkb_comm_init", ctypes.c_int(0), ctypes.c_int(1), z._p(np.zeros(128, dtype=np.uint8)))
    assert "already initialised" in e.value.msg


def test_allgather_single_rank(dev):
    z = dev.z
    src = np.arange(64, dtype=np.uint32)
    d_src, d_dst = z.DeviceBuffer.from_host(src), z.DeviceBuffer(256)
    z.call("zkb_comm_allgather", z._p(d_src), z._p(d_dst), z.sz(256), z._p(0))
    z.call("zkb_sync", z._p(0))
    assert np.array_equal(d_dst.to_host(np.uint32, (64,)), src)


@pytest.mark.parametrize("m,n", [(5, 40), (64, 300)])
def test_commit_sharded_single_rank(dev, m, n):
    z = dev.z
    rng = np.random.Generator(np.random.PCG64(m + n))
    s = rng.integers(0, 1 << 32, size=(n, 8), dtype=np.uint64).astype(np.uint32)
    s[:, 7] %= np.uint32(R.R_MOD >> 224)
    gens = z.DeviceBuffer(144 * n)
    z.call("zkb_g1_mul", z._p(z.DeviceBuffer.from_host(R.g1_pack([R.G1_GEN]))), z.sz(1), z._p(z.DeviceBuffer.from_host(s)), z.sz(n),
           z._p(gens), z._p(0))
    sc = rng.integers(-(1 << 14), 1 << 14, size=m * n, dtype=np.int64).astype(np.int32)
    d_sc = z.DeviceBuffer.from_host(sc)
    a, b = z.DeviceBuffer(144 * m), z.DeviceBuffer(144 * m)
    z.call("zkb_commit_i32", z._p(gens), z.sz(n), z._p(d_sc), z.sz(m * n), z._p(a), z._p(0))
    z.call("zkb_commit_i32_sharded", z._p(gens), z.sz(n), z._p(d_sc), z.sz(m), z.sz(m), z._p(b), z._p(0))
    z.call("zkb_sync", z._p(0))
    # the same points (the Jacobian representative depends on the order the sort's atomics leave)
    pa, pb = R.g1_unpack(a.to_host(np.uint32, (m, 36))), R.g1_unpack(b.to_host(np.uint32, (m, 36)))
    assert all(R.g1_affine(x) == R.g1_affine(y) for x, y in zip(pa, pb))
    with pytest.raises(z.ZkbError) as e:
        z.call("zkb_commit_i32_sharded", z._p(gens), z.sz(n), z._p(d_sc), z.sz(m - 1), z.sz(m), z._p(b), z._p(0))
    assert e.value.code == z.ERR_DIM
    c = z.DeviceBuffer(144 * m)
    z.call("zkb_commit_i32_colsharded", z._p(gens), z.sz(n), z._p(d_sc), z.sz(m), z._p(c), z._p(0))
    z.call("zkb_sync", z._p(0))
    pc = R.g1_unpack(c.to_host(np.uint32, (m, 36)))
    assert all(R.g1_affine(x) == R.g1_affine(y) for x, y in zip(pa, pc))


def test_zkfc_sharded_single_rank(dev):
    z = dev.z
    B, I, O = 8, 64, 32
    rng = np.random.Generator(np.random.PCG64(3))
    X = rng.integers(-3000, 3000, size=(B, I))
    W = rng.integers(-3000, 3000, size=(I, O))
    Y = X @ W
    ub, ui, uo = _rand_fr(rng, 3), _rand_fr(rng, 6), _rand_fr(rng, 5)
    dX, dW, dY = (z.fr_buffer(_ints_to_limbs(t)) for t in (X, W, Y))
    res = []
    for name in ("zkb_zkfc_prove", "zkb_zkfc_prove_sharded"):
        polys, claims = np.zeros((18, 8), dtype=np.uint32), np.zeros((4, 8), dtype=np.uint32)
        z.call(name, z._p(dX), z._p(dW), z._p(dY), z.sz(B), z.sz(I), z.sz(O), z._p(ub), z._p(ui), z._p(uo), z._p(polys), z._p(claims),
               z._p(0))
        res.append((polys, claims))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])


def test_tlookup_sharded_single_rank(dev):
    z = dev.z
    D, N, low = 1 << 12, 1 << 6, -32
    rng = np.random.Generator(np.random.PCG64(9))
    S = rng.integers(low, low + N, size=D)
    counts = np.bincount(S - low, minlength=N)
    dS, dT, dM = (z.fr_buffer(_ints_to_limbs(t)) for t in (S, np.arange(low, low + N), counts))
    alpha, beta, u, v = _rand_fr(rng, 1), _rand_fr(rng, 1), _rand_fr(rng, 12), _rand_fr(rng, 12)
    res = []
    for name in ("zkb_tlookup_prove", "zkb_tlookup_prove_sharded"):
        polys, fin = np.zeros((48, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        z.call(name, z._p(dS), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u), z._p(v), z._p(polys), z._p(fin),
               z._p(0))
        res.append((polys, fin))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])


def test_multi_hadamard_sharded_single_rank(dev):
    import ctypes
    z = dev.z
    K, N = 3, 1 << 11
    rng = np.random.Generator(np.random.PCG64(21))
    Xs = [_rand_fr(rng, N) for _ in range(K)]
    bufs = [z.fr_buffer(x) for x in Xs]
    ptrs = (ctypes.c_void_p * K)(*[b.ptr for b in bufs])
    u, v = _rand_fr(rng, 11), _rand_fr(rng, 11)
    # the claim the proof needs: the product tensor evaluated at u
    prod, claim = z.DeviceBuffer(32 * N), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_fr_mul", z._p(bufs[0]), z._p(bufs[1]), z._p(prod), z.sz(N), z._p(0))
    z.call("zkb_fr_mul", z._p(prod), z._p(bufs[2]), z._p(prod), z.sz(N), z._p(0))
    z.call("zkb_fr_mle_eval", z._p(prod), z.sz(N), z._p(u), z.u32(11), z._p(claim), z._p(0))
    res = []
    for name in ("zkb_multi_hadamard", "zkb_multi_hadamard_sharded"):
        polys, fin = np.zeros((11 * (K + 1), 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        z.call(name, z._p(claim), ptrs, z.u32(K), z.sz(N), z._p(u), z._p(v), z._p(polys), z._p(fin), z._p(0))
        res.append((polys, fin))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])


RANK_SCRIPT = textwrap.dedent('''
    import ctypes, json, os, sys, time
    from pathlib import Path
    import numpy as np
    root = Path(sys.argv[1]); rank = int(sys.argv[2]); world = int(sys.argv[3]); idfile = Path(sys.argv[4])
    sys.path.insert(0, str(root))
    from tests.conftest import load_package
    from oracle import pyref as R
    z = load_package()
    import torch
    torch.cuda.set_device(rank)          # one process per GPU; torch only selects the device here
    ident = np.zeros(128, dtype=np.uint8)
    if rank == 0:
        z.call("zkb_comm_unique_id", z._p(ident))
        tmp = idfile.with_suffix(".tmp"); tmp.write_bytes(ident.tobytes()); tmp.rename(idfile)
    else:
        for _ in range(600):
            if idfile.exists():
                break
            time.sleep(0.1)
        ident = np.frombuffer(idfile.read_bytes(), dtype=np.uint8).copy()
    z.call("zkb_comm_init", ctypes.c_int(rank), ctypes.c_int(world), z._p(ident))

    def limbs(v):
        return R.fr_pack([R.int_to_fr(int(x)) for x in np.asarray(v).reshape(-1)])
    def rand_fr(rng, k):
        v = rng.integers(0, 1 << 32, size=(k, 8), dtype=np.uint64).astype(np.uint32)
        v[:, 7] %= np.uint32(R.R_MOD >> 224)
        return v
    out = {}
    rng = np.random.Generator(np.random.PCG64(77))
    # row commitments: 9 rows over 2 ranks (uneven blocks)
    m, n = 9, 50
    s = rand_fr(rng, n)
    gens = z.DeviceBuffer(144 * n)
    z.call("zkb_g1_mul", z._p(z.DeviceBuffer.from_host(R.g1_pack([R.G1_GEN]))), z.sz(1), z._p(z.DeviceBuffer.from_host(s)), z.sz(n),
           z._p(gens), z._p(0))
    sc = rng.integers(-(1 << 14), 1 << 14, size=(m, n), dtype=np.int64).astype(np.int32)
    base, extra = divmod(m, world)
    b = rank * base + min(rank, extra); e = b + base + (1 if rank < extra else 0)
    whole, gathered = z.DeviceBuffer(144 * m), z.DeviceBuffer(144 * m)
    z.call("zkb_commit_i32", z._p(gens), z.sz(n), z._p(z.DeviceBuffer.from_host(sc.reshape(-1))), z.sz(m * n), z._p(whole), z._p(0))
    z.call("zkb_commit_i32_sharded", z._p(gens), z.sz(n), z._p(z.DeviceBuffer.from_host(np.ascontiguousarray(sc[b:e]).reshape(-1))),
           z.sz(e - b), z.sz(m), z._p(gathered), z._p(0))
    z.call("zkb_sync", z._p(0))
    pts_a = R.g1_unpack(whole.to_host(np.uint32, (m, 36))); pts_b = R.g1_unpack(gathered.to_host(np.uint32, (m, 36)))
    out["commit"] = all(R.g1_affine(p) == R.g1_affine(q) for p, q in zip(pts_a, pts_b))
    # the same matrix split by columns: 50 generators as blocks of 28 and 22
    cols = (0, 28) if rank == 0 else (28, n)
    by_cols = z.DeviceBuffer(144 * m)
    gens_host = gens.to_host(np.uint32, (n, 36))
    z.call("zkb_commit_i32_colsharded", z._p(z.DeviceBuffer.from_host(np.ascontiguousarray(gens_host[cols[0]:cols[1]]))),
           z.sz(cols[1] - cols[0]), z._p(z.DeviceBuffer.from_host(np.ascontiguousarray(sc[:, cols[0]:cols[1]]).reshape(-1))), z.sz(m),
           z._p(by_cols), z._p(0))
    z.call("zkb_sync", z._p(0))
    pts_c = R.g1_unpack(by_cols.to_host(np.uint32, (m, 36)))
    out["commit_cols"] = all(R.g1_affine(p) == R.g1_affine(q) for p, q in zip(pts_a, pts_c))
    # matmul proof
    B, I, O = 8, 64, 32
    X = rng.integers(-3000, 3000, size=(B, I)); W = rng.integers(-3000, 3000, size=(I, O)); Y = X @ W
    ub, ui, uo = rand_fr(rng, 3), rand_fr(rng, 6), rand_fr(rng, 5)
    p0, c0 = np.zeros((18, 8), dtype=np.uint32), np.zeros((4, 8), dtype=np.uint32)
    z.call("zkb_zkfc_prove", z._p(z.fr_buffer(limbs(X))), z._p(z.fr_buffer(limbs(W))), z._p(z.fr_buffer(limbs(Y))), z.sz(B), z.sz(I),
           z.sz(O), z._p(ub), z._p(ui), z._p(uo), z._p(p0), z._p(c0), z._p(0))
    p1, c1 = np.zeros((18, 8), dtype=np.uint32), np.zeros((4, 8), dtype=np.uint32)
    z.call("zkb_zkfc_prove_sharded", z._p(z.fr_buffer(limbs(X[:, rank::world]))), z._p(z.fr_buffer(limbs(W[rank::world, :]))),
           z._p(z.fr_buffer(limbs(Y))), z.sz(B), z.sz(I // world), z.sz(O), z._p(ub), z._p(ui), z._p(uo), z._p(p1), z._p(c1), z._p(0))
    out["zkfc"] = bool(np.array_equal(p0, p1) and np.array_equal(c0, c1))
    # lookup proof
    D, N, low = 1 << 12, 1 << 6, -32
    S = rng.integers(low, low + N, size=D); counts = np.bincount(S - low, minlength=N); T = np.arange(low, low + N)
    alpha, beta, u, v = rand_fr(rng, 1), rand_fr(rng, 1), rand_fr(rng, 12), rand_fr(rng, 12)
    q0, f0 = np.zeros((48, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_tlookup_prove", z._p(z.fr_buffer(limbs(S))), z._p(z.fr_buffer(limbs(T))), z._p(z.fr_buffer(limbs(counts))), z.sz(D), z.sz(N),
           z._p(alpha), z._p(beta), z._p(u), z._p(v), z._p(q0), z._p(f0), z._p(0))
    q1, f1 = np.zeros((48, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_tlookup_prove_sharded", z._p(z.fr_buffer(limbs(S[rank::world]))), z._p(z.fr_buffer(limbs(T[rank::world]))),
           z._p(z.fr_buffer(limbs(counts[rank::world]))), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u), z._p(v), z._p(q1), z._p(f1),
           z._p(0))
    out["tlookup"] = bool(np.array_equal(q0, q1) and np.array_equal(f0, f1))
    # multi-Hadamard sumcheck of three tensors
    K, Nh = 3, 1 << 10
    Xh = [rand_fr(rng, Nh) for _ in range(K)]
    uh, vh, ch = rand_fr(rng, 10), rand_fr(rng, 10), rand_fr(rng, 1)   # an arbitrary claim: only round 0's check sees it
    whole_b = [z.fr_buffer(x) for x in Xh]; share_b = [z.fr_buffer(np.ascontiguousarray(x[rank::world])) for x in Xh]
    res = []
    for name, bufs in (("zkb_multi_hadamard", whole_b), ("zkb_multi_hadamard_sharded", share_b)):
        ptrs = (ctypes.c_void_p * K)(*[b.ptr for b in bufs])
        hp, hf = np.zeros((10 * (K + 1), 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        try:
            z.call(name, z._p(ch), ptrs, z.u32(K), z.sz(Nh), z._p(uh), z._p(vh), z._p(hp), z._p(hf), z._p(0))
            res.append("no error")
        except z.ZkbError as ex:
            res.append((str(ex).split(":")[-1].strip(), hp.tobytes()))
    out["hadamard"] = bool(res[0] == res[1] and res[0] != "no error")
    z.call("zkb_comm_destroy")
    print("RESULT " + json.dumps(out))
''')


def test_two_ranks_match_single_gpu(tmp_path):
    """two processes, one per GPU, over the library's NCCL communicator (NVLS off: plain all-gather)"""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(r), "2", str(tmp_path / "nccl.id")], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    for pr in procs:
        out, _ = pr.communicate(timeout=600)
        assert pr.returncode == 0, out[-2000:]
        line = [l for l in out.splitlines() if l.startswith("RESULT ")][-1]
        assert json.loads(line[7:]) == {"commit": True, "commit_cols": True, "zkfc": True, "tlookup": True, "hadamard": True}, out[-2000:]
