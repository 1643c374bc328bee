"""GPU parity: FrTensor device work against the big-integer oracle (bit-exact)."""
import random

import numpy as np
import pytest

from oracle import pyref as R
from tests.util import Dev, EDGE_FR, rand_fr, rand_small_fr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(zkb):
    return Dev(zkb)


def _binary(dev, name, a, b):
    z = dev.z
    da, db, do = dev.fr(a), dev.fr(b), dev.fr_out(len(a))
    dev.call(name, z._p(da), z._p(db), z._p(do), z.sz(len(a)), z._p(0))
    return dev.read_fr(do, len(a))


def test_elementwise_add_sub_mul(dev):
    rng = random.Random(1)
    a = EDGE_FR + rand_fr(rng, 1000)
    b = list(reversed(EDGE_FR)) + rand_fr(rng, 1000)
    assert _binary(dev, "zkb_fr_add", a, b) == [(x + y) % R.R_MOD for x, y in zip(a, b)]
    assert _binary(dev, "zkb_fr_sub", a, b) == [(x - y) % R.R_MOD for x, y in zip(a, b)]
    assert _binary(dev, "zkb_fr_mul", a, b) == [(x * y) % R.R_MOD for x, y in zip(a, b)]
    assert _binary(dev, "zkb_fr_mont_mul", a, b) == [(x * y * R.FR_RADIX_INV) % R.R_MOD for x, y in zip(a, b)]


def test_all_pairs_of_edge_values(dev):
    a = [x for x in EDGE_FR for _ in EDGE_FR]
    b = [y for _ in EDGE_FR for y in EDGE_FR]
    assert _binary(dev, "zkb_fr_mul", a, b) == [(x * y) % R.R_MOD for x, y in zip(a, b)]
    assert _binary(dev, "zkb_fr_add", a, b) == [(x + y) % R.R_MOD for x, y in zip(a, b)]
    assert _binary(dev, "zkb_fr_sub", a, b) == [(x - y) % R.R_MOD for x, y in zip(a, b)]


def test_unary_and_scalar(dev):
    z = dev.z
    rng = random.Random(2)
    a = EDGE_FR + rand_fr(rng, 300)
    n = len(a)
    da, do = dev.fr(a), dev.fr_out(n)
    dev.call("zkb_fr_neg", z._p(da), z._p(do), z.sz(n), z._p(0))
    assert dev.read_fr(do, n) == [(-x) % R.R_MOD for x in a]
    dev.call("zkb_fr_mont", z._p(da), z._p(do), z.sz(n), z._p(0))
    assert dev.read_fr(do, n) == [x * R.FR_RADIX % R.R_MOD for x in a]
    dev.call("zkb_fr_unmont", z._p(da), z._p(do), z.sz(n), z._p(0))
    assert dev.read_fr(do, n) == [x * R.FR_RADIX_INV % R.R_MOD for x in a]
    for s in (0, 1, R.R_MOD - 1, rng.randrange(R.R_MOD)):
        hs = dev.hfr([s])
        dev.call("zkb_fr_add_scalar", z._p(da), z._p(hs), z._p(do), z.sz(n), z._p(0))
        assert dev.read_fr(do, n) == [(x + s) % R.R_MOD for x in a]
        dev.call("zkb_fr_sub_scalar", z._p(da), z._p(hs), z._p(do), z.sz(n), z._p(0))
        assert dev.read_fr(do, n) == [(x - s) % R.R_MOD for x in a]
        dev.call("zkb_fr_mul_scalar", z._p(da), z._p(hs), z._p(do), z.sz(n), z._p(0))
        assert dev.read_fr(do, n) == [(x * s) % R.R_MOD for x in a]


def test_in_place_and_empty(dev):
    z = dev.z
    a = rand_fr(random.Random(3), 50)
    da = dev.fr(a)
    dev.call("zkb_fr_add", z._p(da), z._p(da), z._p(da), z.sz(50), z._p(0))
    assert dev.read_fr(da, 50) == [2 * x % R.R_MOD for x in a]
    dev.call("zkb_fr_add", z._p(da), z._p(da), z._p(da), z.sz(0), z._p(0))   # empty: no launch, no error


def test_int_conversions(dev):
    z = dev.z
    ints = np.array([0, 1, -1, 2**31 - 1, -2**31, 65536, -65536, 12345, -999], dtype=np.int32)
    n = len(ints)
    di = z.DeviceBuffer.from_host(ints)
    do = dev.fr_out(n)
    dev.call("zkb_fr_from_i32", z._p(di), z._p(do), z.sz(n), z._p(0))
    fr = dev.read_fr(do, n)
    assert fr == [R.int_to_fr(int(v)) for v in ints]
    back = z.DeviceBuffer(4 * n)
    dev.call("zkb_fr_to_i32", z._p(do), z._p(back), z.sz(n), z._p(0))
    assert back.to_host(np.int32, (n,)).tolist() == ints.tolist()
    # values outside the int32 window follow scalar_to_int (fr-tensor.cu:930-934)
    odd = [1 << 31, (1 << 32) - 1, 1 << 32, R.R_MOD - (1 << 31), R.R_MOD - (1 << 32), R.R_MOD - (1 << 40), 1 << 200]
    dodd = dev.fr(odd)
    back = z.DeviceBuffer(4 * len(odd))
    dev.call("zkb_fr_to_i32", z._p(dodd), z._p(back), z.sz(len(odd)), z._p(0))
    assert back.to_host(np.int32, (len(odd),)).tolist() == [R.fr_to_int(v) for v in odd]
    longs = np.array([0, 1, -1, 2**63 - 1, -2**63 + 1, 2**40, -2**40], dtype=np.int64)
    dl = z.DeviceBuffer.from_host(longs)
    do = dev.fr_out(len(longs))
    dev.call("zkb_fr_from_i64", z._p(dl), z._p(do), z.sz(len(longs)), z._p(0))
    assert dev.read_fr(do, len(longs)) == [R.int_to_fr(int(v)) for v in longs]
    back = z.DeviceBuffer(8 * len(longs))
    dev.call("zkb_fr_to_i64", z._p(do), z._p(back), z.sz(len(longs)), z._p(0))
    assert back.to_host(np.int64, (len(longs),)).tolist() == longs.tolist()


def test_float_conversions(dev):
    z = dev.z
    f = np.array([0.0, 0.5, -0.5, 1.25, -1.25, 0.02, -0.02, 3.999999, 100.5], dtype=np.float32)
    df = z.DeviceBuffer.from_host(f)
    do = dev.fr_out(len(f))
    dev.call("zkb_fr_from_f32", z._p(df), z.u64(65536), z._p(do), z.sz(len(f)), z._p(0))
    exp = []
    for v in f:
        x = np.float32(v) * np.float32(65536)           # float product, as float_to_scalar
        xv = float(x)
        exp.append(R.int_to_fr(int(xv + 0.5) if xv >= 0 else int(xv - 0.5)))
    assert dev.read_fr(do, len(f)) == exp
    d = np.array([0.0, 0.49999, -0.5, 1e-3, -123.456], dtype=np.float64)
    dd = z.DeviceBuffer.from_host(d)
    dev.call("zkb_fr_from_f64", z._p(dd), z.u64(1 << 20), z._p(do), z.sz(len(d)), z._p(0))
    exp = []
    for v in d:
        xv = float(v) * float(1 << 20)
        exp.append(R.int_to_fr(int(xv + 0.5) if xv >= 0 else int(xv - 0.5)))
    assert dev.read_fr(do, len(d)) == exp


@pytest.mark.parametrize("n", [1, 2, 255, 256, 257, 5000, 70001])
def test_sum(dev, n):
    z = dev.z
    a = rand_fr(random.Random(n), n)
    out = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_fr_sum", z._p(dev.fr(a)), z.sz(n), z._p(out), z._p(0))
    assert R.fr_unpack(out)[0] == sum(a) % R.R_MOD


@pytest.mark.parametrize("n,k", [(1, 0), (2, 1), (3, 2), (5, 3), (8, 3), (1000, 10), (4096, 12), (5000, 13), (40000, 16)])
def test_mle_eval(dev, n, k):
    z = dev.z
    rng = random.Random(100 + n)
    a, u = rand_fr(rng, n), rand_fr(rng, k)
    out = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_fr_mle_eval", z._p(dev.fr(a)), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z._p(out), z._p(0))
    assert R.fr_unpack(out)[0] == R.mle_eval(a, u)


def test_mle_eval_rejects_bad_dims(dev):
    z = dev.z
    a = rand_fr(random.Random(5), 4)
    out = np.zeros((1, 8), dtype=np.uint32)
    with pytest.raises(z.ZkbError) as e:
        dev.call("zkb_fr_mle_eval", z._p(dev.fr(a)), z.sz(4), z._p(dev.hfr([1, 2, 3])), z.u32(3), z._p(out), z._p(0))
    assert e.value.code == z.ERR_DIM and "Incompatible dimensions" in e.value.msg


@pytest.mark.parametrize("other,cur,window", [(1, 8, 1), (4, 8, 1), (1, 8, 5), (3, 5, 4), (7, 11, 1), (2, 3, 300), (1, 37, 64), (64, 100, 1)])
def test_partial_me(dev, other, cur, window):
    z = dev.z
    rng = random.Random(other * 1000 + cur * 10 + window)
    n = other * cur * window
    k = R.ceil_log2(cur)
    a, u = rand_fr(rng, n), rand_fr(rng, k)
    do = dev.fr_out(other * window)
    dev.call("zkb_fr_partial_me", z._p(dev.fr(a)), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z.sz(cur), z.sz(window), z._p(do), z._p(0))
    assert dev.read_fr(do, other * window) == R.partial_me(a, u, cur, window)


@pytest.mark.parametrize("n,k,window", [(64, 3, 8), (60, 3, 8), (61, 2, 8), (100, 4, 7), (1024, 5, 32), (33, 6, 1)])
def test_partial_me_window(dev, n, k, window):
    z = dev.z
    rng = random.Random(n * 100 + k)
    a, u = rand_fr(rng, n), rand_fr(rng, k)
    exp = R._legacy_partial_me(a, u, window)
    do = dev.fr_out(len(exp) + 8)
    out_n = z.sz(0)
    import ctypes
    dev.call("zkb_fr_partial_me_window", z._p(dev.fr(a)), z.sz(n), z._p(dev.hfr(u)), z.u32(k), z.sz(window), z._p(do),
             ctypes.byref(out_n), z._p(0))
    assert out_n.value == len(exp)
    assert dev.read_fr(do, len(exp)) == exp


@pytest.mark.parametrize("d0,d1", [(1, 1), (1, 8), (8, 1), (4, 8), (5, 7), (33, 100), (128, 300)])
def test_mle_eval_2d(dev, d0, d1):
    z = dev.z
    rng = random.Random(d0 * 1000 + d1)
    a = rand_fr(rng, d0 * d1)
    k0, k1 = R.ceil_log2(d0), R.ceil_log2(d1)
    u0, u1 = rand_fr(rng, k0), rand_fr(rng, k1)
    out = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_fr_mle_eval_2d", z._p(dev.fr(a)), z.sz(d0), z.sz(d1), z._p(dev.hfr(u0)), z.u32(k0),
             z._p(dev.hfr(u1)), z.u32(k1), z._p(out), z._p(0))
    assert R.fr_unpack(out)[0] == R.multi_dim_me(a, [u0, u1], [d0, d1])


def test_pad_transpose_matmul_bias_gather(dev):
    z = dev.z
    rng = random.Random(9)
    rows, last, lp = 5, 11, 16
    a = rand_fr(rng, rows * last)
    do = dev.fr_out(rows * lp)
    dev.call("zkb_fr_pad_last", z._p(dev.fr(a)), z.sz(rows), z.sz(last), z.sz(lp), z._p(dev.hfr([7])), z._p(do), z._p(0))
    exp = []
    for r in range(rows):
        exp += a[r * last:(r + 1) * last] + [7] * (lp - last)
    assert dev.read_fr(do, rows * lp) == exp
    M, N = 37, 70
    a = rand_fr(rng, M * N)
    do = dev.fr_out(M * N)
    dev.call("zkb_fr_transpose", z._p(dev.fr(a)), z.sz(M), z.sz(N), z._p(do), z._p(0))
    assert dev.read_fr(do, M * N) == [a[r * N + c] for c in range(N) for r in range(M)]
    for (M, N, P) in [(1, 1, 1), (3, 5, 7), (33, 17, 40), (64, 64, 64)]:
        x, y = rand_fr(rng, M * N), rand_small_fr(rng, N * P)
        do = dev.fr_out(M * P)
        dev.call("zkb_fr_matmul", z._p(dev.fr(x)), z._p(dev.fr(y)), z._p(do), z.sz(M), z.sz(N), z.sz(P), z._p(0))
        assert dev.read_fr(do, M * P) == R.matmul(x, y, M, N, P)
    zz, bias = rand_fr(rng, 6 * 9), rand_fr(rng, 9)
    dz = dev.fr(zz)
    dev.call("zkb_fr_add_bias", z._p(dz), z._p(dev.fr(bias)), z.sz(6), z.sz(9), z._p(0))
    assert dev.read_fr(dz, 54) == [(zz[i] + bias[i % 9]) % R.R_MOD for i in range(54)]
    vals = rand_fr(rng, 16)
    idx = np.array([rng.randrange(16) for _ in range(100)], dtype=np.uint32)
    do = dev.fr_out(100)
    dev.call("zkb_fr_gather", z._p(z.DeviceBuffer.from_host(idx)), z._p(dev.fr(vals)), z._p(do), z.sz(100), z._p(0))
    assert dev.read_fr(do, 100) == [vals[i] for i in idx]


@pytest.mark.parametrize("n", [1, 7, 2048, 2049, 10000])
def test_inv_shifted(dev, n):
    z = dev.z
    rng = random.Random(n)
    beta = rng.randrange(R.R_MOD)
    a = rand_fr(rng, n)
    a[0] = (-beta) % R.R_MOD            # a + beta == 0 must give 0
    if n > 5:
        a[5] = (-beta) % R.R_MOD
    do = dev.fr_out(n)
    dev.call("zkb_fr_inv_shifted", z._p(dev.fr(a)), z._p(dev.hfr([beta])), z._p(do), z.sz(n), z._p(0))
    assert dev.read_fr(do, n) == [R.fr_inv((x + beta) % R.R_MOD) for x in a]


def test_relu_decomposition(dev):
    """zkReLU's kernel: sign, magnitude, remainder and max(q, 0) of the rescaled value q"""
    z = dev.z
    rng = random.Random(12)
    vals = [0, 1, -1, 32767, 32768, -32768, -32769, 65536, -65536, 98304, -98304, 2**40 + 12345, -(2**40) - 77]
    vals += [rng.randrange(-2**45, 2**45) for _ in range(300)]
    for sf in (1 << 16, 1 << 20, 3):
        x = [R.int_to_fr(v) for v in vals]
        outs = [dev.fr_out(len(x)) for _ in range(4)]
        dev.call("zkb_relu_decomp", z._p(dev.fr(x)), z.u64(sf), *[z._p(o) for o in outs], z.sz(len(x)), z._p(0))
        exp = R.relu_decomp(x, sf)
        for got, e in zip(outs, exp):
            assert dev.read_fr(got, len(x)) == e
        for v, sg, mg, rm, rs in zip(vals, *exp):
            q = (v - R.fr_to_long(rm)) // sf
            assert (sg, mg, R.fr_to_long(rs)) == (1 if q >= 0 else 0, abs(q), max(q, 0))


def test_rescale(dev):
    z = dev.z
    rng = random.Random(11)
    vals = [0, 1, -1, 32767, 32768, 32769, -32767, -32768, -32769, 65536, -65536, 98304, -98304, 2**40 + 12345, -(2**40) - 77]
    vals += [rng.randrange(-2**45, 2**45) for _ in range(500)]
    for sf in (1 << 16, 1 << 20, 3):
        x = [R.int_to_fr(v) for v in vals]
        do, dr = dev.fr_out(len(x)), dev.fr_out(len(x))
        dev.call("zkb_rescale", z._p(dev.fr(x)), z.u64(sf), z._p(do), z._p(dr), z.sz(len(x)), z._p(0))
        eo, er = R.rescale(x, sf)
        assert dev.read_fr(do, len(x)) == eo
        assert dev.read_fr(dr, len(x)) == er
        # the defining identity: x = out * sf + rem, rem in [-sf/2, sf/2)
        for v, o, r_ in zip(vals, eo, er):
            assert R.fr_to_long(o) * sf + R.fr_to_long(r_) == v
