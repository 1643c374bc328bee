"""GPU parity: sumcheck provers against the big-integer oracle (bit-exact transcripts)."""
import random

import numpy as np
import pytest

from oracle import pyref as R
from tests.util import Dev, rand_fr, rand_small_fr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(zkb):
    return Dev(zkb)


def _zkip(dev, claim, a, b, u):
    z = dev.z
    k = len(u)
    polys = np.zeros((max(3 * k, 1), 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_zkip", z._p(dev.hfr([claim])), z._p(dev.fr(a)), z._p(dev.fr(b)), z.sz(len(a)), z._p(dev.hfr(u)),
             z.u32(k), z._p(polys), z._p(final), z._p(0))
    p = R.fr_unpack(polys)[:3 * k]
    return [p[3 * i:3 * i + 3] for i in range(k)], R.fr_unpack(final)[0]


@pytest.mark.parametrize("n", [2, 3, 4, 7, 8, 100, 1024, 5000, 16384])
def test_zkip(dev, n):
    rng = random.Random(n)
    a, b = rand_fr(rng, n), rand_fr(rng, n)
    u = rand_fr(rng, R.ceil_log2(n))
    claim = sum(x * y for x, y in zip(a, b)) % R.R_MOD
    proof = []
    exp_final = R.zkip(claim, a, b, u, proof)
    polys, final = _zkip(dev, claim, a, b, u)
    assert polys == proof
    assert final == exp_final


def test_zkip_wrong_claim_fails(dev):
    z = dev.z
    rng = random.Random(77)
    a, b = rand_fr(rng, 64), rand_fr(rng, 64)
    u = rand_fr(rng, 6)
    claim = (sum(x * y for x, y in zip(a, b)) + 1) % R.R_MOD
    with pytest.raises(z.ZkbError) as e:
        _zkip(dev, claim, a, b, u)
    assert e.value.code == z.ERR_VERIFY and e.value.msg == "claim != p(0) + p(1)"


def test_zkip_no_rounds_returns_claim(dev):
    polys, final = _zkip(dev, 12345, [5], [7], [])
    assert polys == [] and final == 12345


@pytest.mark.parametrize("B,I,O", [(1, 1, 8), (1, 8, 1), (4, 8, 16), (3, 5, 7), (16, 33, 20), (128, 64, 96)])
def test_zkfc_prove(dev, B, I, O):
    z = dev.z
    rng = random.Random(B * 10000 + I * 100 + O)
    X, W = rand_small_fr(rng, B * I), rand_small_fr(rng, I * O)
    Y = R.matmul(X, W, B, I, O)
    ub, ui, uo = rand_fr(rng, R.ceil_log2(B)), rand_fr(rng, R.ceil_log2(I)), rand_fr(rng, R.ceil_log2(O))
    exp = R.zkfc_prove(X, W, Y, B, I, O, ub, ui, uo)
    kI = len(ui)
    polys = np.zeros((max(3 * kI, 1), 8), dtype=np.uint32)
    claims = np.zeros((4, 8), dtype=np.uint32)
    dev.call("zkb_zkfc_prove", z._p(dev.fr(X)), z._p(dev.fr(W)), z._p(dev.fr(Y)), z.sz(B), z.sz(I), z.sz(O),
             z._p(dev.hfr(ub)), z._p(dev.hfr(ui)), z._p(dev.hfr(uo)), z._p(polys), z._p(claims), z._p(0))
    p = R.fr_unpack(polys)[:3 * kI]
    assert [p[3 * i:3 * i + 3] for i in range(kI)] == exp["proof"]
    c = R.fr_unpack(claims)
    assert c == [exp["claim"], exp["final_claim"], exp["claim_x"], exp["claim_w"]]


def test_zkfc_prove_rejects_wrong_output(dev):
    z = dev.z
    rng = random.Random(3)
    B, I, O = 4, 8, 8
    X, W = rand_small_fr(rng, B * I), rand_small_fr(rng, I * O)
    Y = R.matmul(X, W, B, I, O)
    Y[3] = (Y[3] + 1) % R.R_MOD
    ub, ui, uo = rand_fr(rng, 2), rand_fr(rng, 3), rand_fr(rng, 3)
    polys = np.zeros((9, 8), dtype=np.uint32)
    claims = np.zeros((4, 8), dtype=np.uint32)
    with pytest.raises(z.ZkbError) as e:
        dev.call("zkb_zkfc_prove", z._p(dev.fr(X)), z._p(dev.fr(W)), z._p(dev.fr(Y)), z.sz(B), z.sz(I), z.sz(O),
                 z._p(dev.hfr(ub)), z._p(dev.hfr(ui)), z._p(dev.hfr(uo)), z._p(polys), z._p(claims), z._p(0))
    assert e.value.code == z.ERR_VERIFY


@pytest.mark.parametrize("N,D", [(4, 8), (3, 5), (8, 1), (1, 16), (32, 128), (5, 64), (2, 1000)])
def test_zkip_stacked(dev, N, D):
    """the fused stack rounds + zkip over D against the restatement of zkfc.cu:187-228"""
    z = dev.z
    rng = random.Random(N * 1000 + D)
    A, B = rand_fr(rng, N * D), rand_fr(rng, N * D)
    kN, kD = R.ceil_log2(N), R.ceil_log2(D)
    uN, vN, uD = rand_fr(rng, kN), rand_fr(rng, kN), rand_fr(rng, kD)
    # the claim the stacked prover starts from: sum_n eq(uN; n) <A_n, B_n>
    weights = [1] * N
    for n in range(N):
        for j, x in enumerate(uN):
            weights[n] = weights[n] * (x if (n >> j) & 1 else (1 - x)) % R.R_MOD
    claim = sum(weights[n] * sum(A[n * D + d] * B[n * D + d] for d in range(D)) for n in range(N)) % R.R_MOD
    proof = []
    exp_final = R.zkip_stacked(claim, A, B, uN, uD, vN, N, D, proof)
    polys, final = np.zeros((max(3 * (kN + kD), 1), 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_zkip_stacked", z._p(dev.hfr([claim])), z._p(dev.fr(A)), z._p(dev.fr(B)), z.sz(N), z.sz(D), z._p(dev.hfr(uN)),
             z._p(dev.hfr(vN)), z.u32(kN), z._p(dev.hfr(uD)), z.u32(kD), z._p(polys), z._p(final), z._p(0))
    got = R.fr_unpack(polys)[:3 * (kN + kD)]
    assert [got[3 * i:3 * i + 3] for i in range(kN + kD)] == proof
    assert R.fr_unpack(final)[0] == exp_final
    if kN:
        with pytest.raises(z.ZkbError) as e:
            dev.call("zkb_zkip_stacked", z._p(dev.hfr([(claim + 1) % R.R_MOD])), z._p(dev.fr(A)), z._p(dev.fr(B)), z.sz(N), z.sz(D),
                     z._p(dev.hfr(uN)), z._p(dev.hfr(vN)), z.u32(kN), z._p(dev.hfr(uD)), z.u32(kD), z._p(polys), z._p(final), z._p(0))
        assert e.value.code == z.ERR_VERIFY and "claim != q(0) + q(1)" in e.value.msg


def _tlookup(dev, S, table, m, alpha, beta, u, v, indices=None):
    """indices: None = zkb_tlookup_prove; a list = zkb_tlookup_prove_indexed with those claimed table positions"""
    z = dev.z
    D, N = len(S), len(table)
    kD = R.ceil_log2(D)
    polys = np.zeros((max(4 * kD, 1), 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    if indices is None:
        dev.call("zkb_tlookup_prove", z._p(dev.fr(S)), z._p(dev.fr(table)), z._p(dev.fr(m)), z.sz(D), z.sz(N),
                 z._p(dev.hfr([alpha])), z._p(dev.hfr([beta])), z._p(dev.hfr(u)), z._p(dev.hfr(v)), z._p(polys), z._p(final), z._p(0))
    else:
        d_idx = z.DeviceBuffer.from_host(np.array(indices, dtype=np.uint32))
        dev.call("zkb_tlookup_prove_indexed", z._p(dev.fr(S)), z._p(d_idx), z._p(dev.fr(table)), z._p(dev.fr(m)), z.sz(D), z.sz(N),
                 z._p(dev.hfr([alpha])), z._p(dev.hfr([beta])), z._p(dev.hfr(u)), z._p(dev.hfr(v)), z._p(polys), z._p(final), z._p(0))
    p = R.fr_unpack(polys)[:4 * kD]
    return [p[4 * i:4 * i + 4] for i in range(kD)], R.fr_unpack(final)[0]


@pytest.mark.parametrize("D,N,low", [(8, 8, -4), (16, 4, 0), (64, 8, -4), (1024, 16, -8), (8192, 256, -128), (32768, 8192, -4096), (4, 1, 3)])
def test_tlookup_prove(dev, D, N, low):
    rng = random.Random(D * 31 + N)
    table = R.range_table(low, N)
    vals = [R.int_to_fr(rng.randrange(low, low + N)) for _ in range(D)]
    idx = R.range_indices(vals, low)
    m = R.tlookup_prep(idx, N)
    alpha, beta = rng.randrange(R.R_MOD), rng.randrange(R.R_MOD)
    k = R.ceil_log2(D)
    u, v = rand_fr(rng, k), rand_fr(rng, k)
    exp_polys = []
    exp = R.tlookup_prove(vals, table, m, alpha, beta, u, v, exp_polys)
    polys, final = _tlookup(dev, vals, table, m, alpha, beta, u, v)
    assert [[c % R.R_MOD for c in (p + [0, 0, 0, 0])[:4]] for p in exp_polys] == polys
    assert final == exp
    # with the table positions given (inverses read from the table's), and with positions that are
    # wrong, out of range or all the same (every value then inverted on its own): the same transcript
    wrong = [rng.randrange(0, 2 * N) for _ in range(D)]
    for indices in (idx, wrong, [0] * D, [i if k % 3 else 0xFFFFFFFF for k, i in enumerate(idx)]):
        p2, f2 = _tlookup(dev, vals, table, m, alpha, beta, u, v, indices)
        assert p2 == polys and f2 == final


def test_tlookup_value_equal_to_minus_beta(dev):
    """S + beta = 0 for some entries: the inverse is taken as 0 (tlookup.cu:50-62) on every path, so the
    plain and the indexed prover agree with each other and with the oracle - whether the proof passes or not"""
    z = dev.z
    rng = random.Random(77)
    D, N, low = 256, 16, -8
    table = R.range_table(low, N)
    vals = [R.int_to_fr(rng.randrange(low, low + N)) for _ in range(D)]
    idx = R.range_indices(vals, low)
    m = R.tlookup_prep(idx, N)
    alpha, beta = rng.randrange(R.R_MOD), (-vals[5]) % R.R_MOD
    u, v = rand_fr(rng, 8), rand_fr(rng, 8)
    outcomes = []
    for indices in (None, idx):
        try:
            outcomes.append(_tlookup(dev, vals, table, m, alpha, beta, u, v, indices))
        except z.ZkbError as e:
            outcomes.append(("error", e.msg))
    try:
        exp_polys = []
        exp = R.tlookup_prove(vals, table, m, alpha, beta, u, v, exp_polys)
        oracle = ([[c % R.R_MOD for c in (p + [0, 0, 0, 0])[:4]] for p in exp_polys], exp)
    except Exception as e:      # the oracle raises the reference's message
        oracle = ("error", str(e))
    assert outcomes[0] == outcomes[1]
    if oracle[0] == "error":
        assert outcomes[0][0] == "error" and oracle[1] in outcomes[0][1]
    else:
        assert outcomes[0] == oracle


def test_tlookup_bad_multiplicities_fail(dev):
    z = dev.z
    rng = random.Random(5)
    D, N, low = 64, 8, 0
    table = R.range_table(low, N)
    vals = [R.int_to_fr(rng.randrange(low, low + N)) for _ in range(D)]
    m = R.tlookup_prep(R.range_indices(vals, low), N)
    m[2] = (m[2] + 1) % R.R_MOD
    u, v = rand_fr(rng, 6), rand_fr(rng, 6)
    with pytest.raises(z.ZkbError) as e:
        _tlookup(dev, vals, table, m, rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), u, v)
    assert e.value.code == z.ERR_VERIFY and "claim != p(0) + p(1)" in e.value.msg


def test_tlookup_helpers(dev):
    z = dev.z
    rng = random.Random(6)
    low, length, size = -5, 11, 16
    dt = dev.fr_out(size)
    dev.call("zkb_tlookup_range_table", z.i32(low), z.sz(length), z.sz(size), z._p(dt), z._p(0))
    assert dev.read_fr(dt, size) == R.range_table(low, length)
    vals = [R.int_to_fr(rng.randrange(low, low + length)) for _ in range(300)]
    di = z.DeviceBuffer(4 * 300)
    dev.call("zkb_tlookup_range_indices", z._p(dev.fr(vals)), z.i32(low), z._p(di), z.sz(300), z._p(0))
    idx = di.to_host(np.uint32, (300,)).tolist()
    assert idx == R.range_indices(vals, low)
    dm = dev.fr_out(size)
    dev.call("zkb_tlookup_prep", z._p(di), z.sz(300), z.sz(size), z._p(dm), z._p(0))
    assert dev.read_fr(dm, size) == R.tlookup_prep(idx, size)


@pytest.mark.parametrize("K,N", [(1, 8), (2, 2), (2, 64), (3, 1024), (4, 256), (2, 16384), (6, 32)])
def test_multi_hadamard(dev, K, N):
    z = dev.z
    import ctypes
    rng = random.Random(K * 100000 + N)
    Xs = [rand_fr(rng, N) for _ in range(K)]
    k = R.ceil_log2(N)
    u, v = rand_fr(rng, k), rand_fr(rng, k)
    prod = [1] * N
    for X in Xs:
        prod = [p * x % R.R_MOD for p, x in zip(prod, X)]
    claim = R.mle_eval(prod, u)
    proof = []
    exp = R.multi_hadamard_sumchecks(claim, Xs, u, v, proof)
    bufs = [dev.fr(X) for X in Xs]
    ptrs = (ctypes.c_void_p * K)(*[b.ptr for b in bufs])
    polys = np.zeros((k * (K + 1), 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_multi_hadamard", z._p(dev.hfr([claim])), ptrs, z.u32(K), z.sz(N), z._p(dev.hfr(u)), z._p(dev.hfr(v)),
             z._p(polys), z._p(final), z._p(0))
    p = R.fr_unpack(polys)
    assert [p[i * (K + 1):(i + 1) * (K + 1)] for i in range(k)] == proof
    assert R.fr_unpack(final)[0] == exp


@pytest.mark.parametrize("n", [1, 2, 3, 5, 8, 100, 1000, 4097, 20000])
def test_legacy_sumchecks(dev, n):
    z = dev.z
    rng = random.Random(n)
    k = R.ceil_log2(n)
    a, b = rand_fr(rng, n), rand_fr(rng, n)
    u, v = rand_fr(rng, k), rand_fr(rng, k)
    if k >= 1:   # with no challenges the reference's own size check shifts by -1
        out = np.zeros((3 * k + 2, 8), dtype=np.uint32)
        dev.call("zkb_hadamard_product_sumcheck", z._p(dev.fr(a)), z._p(dev.fr(b)), z.sz(n), z._p(dev.hfr(u)), z._p(dev.hfr(v)),
                 z.u32(k), z._p(out), z._p(0))
        assert R.fr_unpack(out) == R.hadamard_product_sumcheck(a, b, u, v)
    out = np.zeros((3 * k + 2, 8), dtype=np.uint32)
    dev.call("zkb_inner_product_sumcheck", z._p(dev.fr(a)), z._p(dev.fr(b)), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z._p(out), z._p(0))
    assert R.fr_unpack(out) == R.inner_product_sumcheck(a, b, u)
    out = np.zeros((3 * k + 1, 8), dtype=np.uint32)
    dev.call("zkb_binary_sumcheck", z._p(dev.fr(a)), z.sz(n), z._p(dev.hfr(u)), z._p(dev.hfr(v)), z.u32(k), z._p(out), z._p(0))
    assert R.fr_unpack(out) == R.binary_sumcheck(a, u, v)
