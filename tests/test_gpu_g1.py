"""GPU parity: G1 tensors, commitments and openings against the big-integer
oracle.  G1 results are compared on the affine point, Fr results bit for bit."""
import ctypes
import random

import numpy as np
import pytest

from oracle import pyref as R
from tests.util import Dev, affine_eq, rand_fr, seeded_generators

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(zkb):
    return Dev(zkb)


@pytest.fixture(scope="module")
def gens():
    return seeded_generators(40, 1234)


def _rand_jac(rng, pts):
    """re-randomise the Jacobian representative of each point"""
    out = []
    for (x, y, z) in pts:
        if z == 0:
            out.append((x, y, z))
            continue
        l = rng.randrange(1, R.Q_MOD)
        out.append((x * l * l % R.Q_MOD, y * l * l * l % R.Q_MOD, z * l % R.Q_MOD))
    return out


def test_add_sub_neg_double_and_special_cases(dev, gens):
    z = dev.z
    rng = random.Random(1)
    a = _rand_jac(rng, gens[:16])
    b = _rand_jac(rng, gens[16:32])
    # special cases: identity operands, P + P, P + (-P)
    a += [R.G1_ZERO, gens[0], R.G1_ZERO, gens[3], gens[4]]
    b += [gens[1], R.G1_ZERO, R.G1_ZERO, _rand_jac(rng, [gens[3]])[0], R.g1_neg(_rand_jac(rng, [gens[4]])[0])]
    n = len(a)
    da, db, do = dev.g1(a), dev.g1(b), z.DeviceBuffer(144 * n)
    dev.call("zkb_g1_add", z._p(da), z._p(db), z._p(do), z.sz(n), z._p(0))
    out = dev.read_g1(do, n)
    for i in range(n):
        assert affine_eq(out[i], R.g1_add(a[i], b[i])), i
        assert R.g1_on_curve(out[i])
    dev.call("zkb_g1_sub", z._p(da), z._p(db), z._p(do), z.sz(n), z._p(0))
    out = dev.read_g1(do, n)
    for i in range(n):
        assert affine_eq(out[i], R.g1_add(a[i], R.g1_neg(b[i]))), i
    dev.call("zkb_g1_neg", z._p(da), z._p(do), z.sz(n), z._p(0))
    out = dev.read_g1(do, n)
    for i in range(n):
        assert affine_eq(out[i], R.g1_neg(a[i]))
    h = R.g1_pack([gens[7]])
    dev.call("zkb_g1_add_scalar", z._p(da), z._p(h), z._p(do), z.sz(n), z._p(0))
    out = dev.read_g1(do, n)
    for i in range(n):
        assert affine_eq(out[i], R.g1_add(a[i], gens[7]))


def test_affine_round_trip_and_fill(dev, gens):
    z = dev.z
    rng = random.Random(2)
    a = _rand_jac(rng, gens[:10]) + [R.G1_ZERO]
    n = len(a)
    daff = z.DeviceBuffer(96 * n)
    dev.call("zkb_g1_to_affine", z._p(dev.g1(a)), z._p(daff), z.sz(n), z._p(0))
    aff = daff.to_host(np.uint32, (n, 24))
    for i in range(n):
        x = R.limbs_to_int(aff[i, :12]) * R.FQ_RADIX_INV % R.Q_MOD
        y = R.limbs_to_int(aff[i, 12:]) * R.FQ_RADIX_INV % R.Q_MOD
        exp = R.g1_affine(a[i])
        assert (x, y) == (exp if exp is not None else (0, 0))
    dj = z.DeviceBuffer(144 * n)
    dev.call("zkb_g1_from_affine", z._p(daff), z._p(dj), z.sz(n), z._p(0))
    back = dev.read_g1(dj, n)
    for i in range(n - 1):
        assert affine_eq(back[i], a[i]) and back[i][2] == 1
    dev.call("zkb_g1_fill", z._p(dj), z._p(R.g1_pack([gens[2]])), z.sz(n), z._p(0))
    assert all(p == gens[2] for p in dev.read_g1(dj, n))


def test_scalar_mul_sum_rowwise(dev, gens):
    z = dev.z
    rng = random.Random(3)
    ng = 6
    ks = [0, 1, 2, R.R_MOD - 1, (1 << 255) - 19, 5] + rand_fr(rng, 12)
    n = len(ks)
    do = z.DeviceBuffer(144 * n)
    dev.call("zkb_g1_mul", z._p(dev.g1(gens[:ng])), z.sz(ng), z._p(dev.fr(ks)), z.sz(n), z._p(do), z._p(0))
    out = dev.read_g1(do, n)
    for i in range(n):
        assert affine_eq(out[i], R.g1_mul(gens[i % ng], ks[i])), i
    for cnt in (1, 2, 33, 40):
        hs = np.zeros((1, 36), dtype=np.uint32)
        dev.call("zkb_g1_sum", z._p(dev.g1(gens[:cnt])), z.sz(cnt), z._p(hs), z._p(0))
        assert affine_eq(R.g1_unpack(hs)[0], R.g1_sum(gens[:cnt]))
    rows, cols = 5, 8
    do = z.DeviceBuffer(144 * rows)
    dev.call("zkb_g1_rowwise_sum", z._p(dev.g1(gens[:rows * cols])), z.sz(rows), z.sz(cols), z._p(do), z._p(0))
    out = dev.read_g1(do, rows)
    for r in range(rows):
        assert affine_eq(out[r], R.g1_sum(gens[r * cols:(r + 1) * cols]))


@pytest.mark.parametrize("n", [1, 2, 5, 8])
def test_g1_mle_eval(dev, gens, n):
    z = dev.z
    rng = random.Random(n)
    k = R.ceil_log2(n)
    u = rand_fr(rng, k)
    hs = np.zeros((1, 36), dtype=np.uint32)
    dev.call("zkb_g1_mle_eval", z._p(dev.g1(gens[:n])), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z._p(hs), z._p(0))
    # reference quirk (g1-tensor.cu:491): the challenge is un-Montgomeried before its bits are used
    t = list(gens[:n])
    for x in u:
        xb = x * R.FR_RADIX_INV % R.R_MOD
        nt = []
        for g in range((len(t) + 1) // 2):
            if 2 * g + 1 < len(t):
                nt.append(R.g1_add(t[2 * g], R.g1_mul(R.g1_add(t[2 * g + 1], R.g1_neg(t[2 * g])), xb)))
            else:
                nt.append(R.g1_add(t[2 * g], R.g1_neg(R.g1_mul(t[2 * g], xb))))
        t = nt
    assert affine_eq(R.g1_unpack(hs)[0], t[0])


@pytest.mark.parametrize("m,n,bits", [(1, 1, 8), (1, 40, 14), (3, 17, 14), (4, 40, 31), (2, 33, 5), (33, 8, 13)])
def test_commit_int(dev, m, n, bits):
    z = dev.z
    rng = random.Random(m * 1000 + n + bits)
    g = seeded_generators(n, 99)[:n] if n > 40 else seeded_generators(40, 1234)[:n]
    ints = [rng.randrange(-(1 << bits), 1 << bits) for _ in range(m * n)]
    ints[0] = 0
    if bits == 31:
        ints[1], ints[2] = -(1 << 31), (1 << 31) - 1
    exp = R.commit_int(g, [R.int_to_fr(v) for v in ints])
    dg = dev.g1(g)
    do = z.DeviceBuffer(144 * m)
    dev.call("zkb_commit_int", z._p(dg), z.sz(n), z._p(dev.fr([R.int_to_fr(v) for v in ints])), z.sz(m * n), z._p(do), z._p(0))
    out = dev.read_g1(do, m)
    for r in range(m):
        assert affine_eq(out[r], exp[r]) and R.g1_on_curve(out[r]), r
    di = z.DeviceBuffer.from_host(np.array(ints, dtype=np.int32))
    dev.call("zkb_commit_i32", z._p(dg), z.sz(n), z._p(di), z.sz(m * n), z._p(do), z._p(0))
    out = dev.read_g1(do, m)
    for r in range(m):
        assert affine_eq(out[r], exp[r]), r
    # both algorithms by name: buckets (1) and combination tables (2)
    for method in (1, 2):
        dev.call("zkb_commit_i32_method", z._p(dg), z.sz(n), z._p(di), z.sz(m * n), z._p(do), ctypes.c_int(method), z._p(0))
        out = dev.read_g1(do, m)
        for r in range(m):
            assert affine_eq(out[r], exp[r]) and R.g1_on_curve(out[r]), (method, r)
    hout = np.zeros((m, 36), dtype=np.uint32)
    dev.call("zkb_commit_i32_host", z._p(R.g1_pack(g)), z.sz(n), z._p(np.array(ints, dtype=np.int32)), z.sz(m * n), z._p(hout), z._p(0))
    out = R.g1_unpack(hout)
    for r in range(m):
        assert affine_eq(out[r], exp[r]), r


def test_commit_int_rejects_bad_shape(dev, gens):
    z = dev.z
    with pytest.raises(z.ZkbError) as e:
        dev.call("zkb_commit_int", z._p(dev.g1(gens[:4])), z.sz(4), z._p(dev.fr([1] * 6)), z.sz(6), z._p(z.DeviceBuffer(144 * 2)), z._p(0))
    assert e.value.code == z.ERR_DIM and "Commitment::commit_int - Incompatible dimensions" in e.value.msg


def test_commit_duplicate_and_identity_generators(dev, gens):
    """P + P, P + (-P) and identity generators inside one bucket"""
    z = dev.z
    g = [gens[0], gens[0], R.g1_neg(gens[0]), R.G1_ZERO, gens[1], gens[1]]
    ints = [3, 3, 3, 9, 5, -5, 1, 1, 1, 0, 0, 0]
    exp = R.commit_int(g, [R.int_to_fr(v) for v in ints])
    do = z.DeviceBuffer(144 * 2)
    dev.call("zkb_commit_int", z._p(dev.g1(g)), z.sz(6), z._p(dev.fr([R.int_to_fr(v) for v in ints])), z.sz(12), z._p(do), z._p(0))
    out = dev.read_g1(do, 2)
    assert affine_eq(out[0], exp[0]) and affine_eq(out[1], exp[1])
    di = z.DeviceBuffer.from_host(np.array(ints, dtype=np.int32))
    for method in (1, 2):
        dev.call("zkb_commit_i32_method", z._p(dev.g1(g)), z.sz(6), z._p(di), z.sz(12), z._p(do), ctypes.c_int(method), z._p(0))
        out = dev.read_g1(do, 2)
        assert affine_eq(out[0], exp[0]) and affine_eq(out[1], exp[1]), method


def test_commit_tables_special_points(dev, gens):
    """combination tables whose entries meet P + P, P + (-P) and the identity while they are built:
    equal, opposite and identity generators inside one group of four, every digit from -4 to 3"""
    z = dev.z
    P, Q = gens[0], gens[1]
    g = [P, P, R.g1_neg(P), R.G1_ZERO, Q, R.g1_neg(Q), Q, P, R.G1_ZERO, R.G1_ZERO, R.G1_ZERO, R.G1_ZERO, Q]
    n = len(g)
    rng = random.Random(5)
    rows = [[rng.randrange(-4, 4) for _ in range(n)] for _ in range(6)]
    rows.append([3] * n)
    rows.append([-4] * n)
    rows.append([0] * n)
    rows.append([rng.randrange(-14000, 14000) for _ in range(n)])
    ints = [v for r in rows for v in r]
    m = len(rows)
    exp = R.commit_int(g, [R.int_to_fr(v) for v in ints])
    do = z.DeviceBuffer(144 * m)
    di = z.DeviceBuffer.from_host(np.array(ints, dtype=np.int32))
    for method in (1, 2):
        dev.call("zkb_commit_i32_method", z._p(dev.g1(g)), z.sz(n), z._p(di), z.sz(m * n), z._p(do), ctypes.c_int(method), z._p(0))
        out = dev.read_g1(do, m)
        for r in range(m):
            assert affine_eq(out[r], exp[r]), (method, r)


def test_commit_method_rejects_unknown(dev, gens):
    z = dev.z
    di = z.DeviceBuffer.from_host(np.array([1, 2, 3, 4], dtype=np.int32))
    with pytest.raises(z.ZkbError) as e:
        dev.call("zkb_commit_i32_method", z._p(dev.g1(gens[:4])), z.sz(4), z._p(di), z.sz(4), z._p(z.DeviceBuffer(144)), ctypes.c_int(7), z._p(0))
    assert e.value.code == z.ERR_ARG


def curve_points_outside_the_subgroup(count: int, seed: int) -> list:
    """points of E(Fq): y^2 = x^3 + 4 that are not in the order-r subgroup (the cofactor is large, so a random
    curve point almost never is); Jacobian triples with Z = 1"""
    rng = random.Random(seed)
    out = []
    while len(out) < count:
        x = rng.randrange(R.Q_MOD)
        rhs = (x * x * x + 4) % R.Q_MOD
        y = pow(rhs, (R.Q_MOD + 1) // 4, R.Q_MOD)          # q = 3 mod 4
        if y * y % R.Q_MOD != rhs:
            continue
        P = (x, y, 1)
        if R.g1_affine(R.g1_mul(P, R.R_MOD)) is not None:
            out.append(P)
    return out


@pytest.mark.parametrize("n,k", [(1, 1), (2, 1), (4, 2), (5, 3), (8, 3), (6, 2)])
def test_me_open_with_generators_outside_the_subgroup(dev, gens, n, k):
    """a generator file need not hold points of order r: the opening then follows the reference's own arithmetic
    (me_open_step, commitment.cu:79-109: scalars and challenges as 256 raw bits) and returns its group elements"""
    z = dev.z
    rng = random.Random(n * 11 + k)
    wild = curve_points_outside_the_subgroup(n, 100 + n)
    # a mixed set as well: one stray point among proper generators is enough to leave the fast path
    for g in (wild, [wild[0]] + list(gens[:n - 1])):
        t, u = rand_fr(rng, n), rand_fr(rng, k)
        proof = []
        exp = R.me_open(t, g, u, proof)
        hp = np.zeros((3 * k + 1, 36), dtype=np.uint32)
        ho = np.zeros((1, 8), dtype=np.uint32)
        dev.call("zkb_me_open", z._p(dev.fr(t)), z._p(dev.g1(g)), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z._p(hp), z._p(ho), z._p(0))
        assert R.fr_unpack(ho)[0] == exp
        got = R.g1_unpack(hp)
        assert len(got) == len(proof)
        for a, b in zip(got, proof):
            assert affine_eq(a, b)


@pytest.mark.parametrize("m,n", [(1, 3), (2, 8)])
def test_commit_full_width(dev, gens, m, n):
    z = dev.z
    rng = random.Random(m * 10 + n)
    sc = rand_fr(rng, m * n)
    sc[0] = 0
    sc[1] = R.R_MOD - 1
    exp = R.commit(gens[:n], sc)
    do = z.DeviceBuffer(144 * m)
    dev.call("zkb_commit", z._p(dev.g1(gens[:n])), z.sz(n), z._p(dev.fr(sc)), z.sz(m * n), z._p(do), z._p(0))
    out = dev.read_g1(do, m)
    for r in range(m):
        assert affine_eq(out[r], exp[r]), r


@pytest.mark.parametrize("n,k", [(1, 0), (2, 1), (4, 2), (5, 3), (8, 3), (3, 4), (1, 2), (8, 2)])
def test_me_open(dev, gens, n, k):
    z = dev.z
    rng = random.Random(n * 7 + k)
    t, u = rand_fr(rng, n), rand_fr(rng, k)
    proof = []
    exp = R.me_open(t, gens[:n], u, proof)
    hp = np.zeros((3 * k + 1, 36), dtype=np.uint32)
    ho = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_me_open", z._p(dev.fr(t)), z._p(dev.g1(gens[:n])), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z._p(hp), z._p(ho), z._p(0))
    assert R.fr_unpack(ho)[0] == exp
    got = R.g1_unpack(hp)
    assert len(got) == len(proof)
    for a, b in zip(got, proof):
        assert affine_eq(a, b)
