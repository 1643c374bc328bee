"""GPU parity at sizes the Python oracle cannot reach: against the C++ oracle, and
through size-independent properties (linearity of the commitment, the provers'
own verifier equations) at larger sizes."""
import ctypes
import random

import numpy as np
import pytest

from oracle import cpporacle as C
from oracle import pyref as R
from tests.util import Dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(zkb):
    return Dev(zkb)


def gpu_generators(dev, n, seed):
    """n generators s_i * G made on the device (checked against the oracle in test_gpu_g1)"""
    z = dev.z
    rng = np.random.Generator(np.random.PCG64(seed))
    s = rng.integers(0, 1 << 32, size=(n, 8), dtype=np.uint64).astype(np.uint32)
    s[:, 7] %= np.uint32(R.R_MOD >> 224)
    out = z.DeviceBuffer(144 * n)
    g1 = z.DeviceBuffer.from_host(R.g1_pack([R.G1_GEN]))
    dev.call("zkb_g1_mul", z._p(g1), z.sz(1), z._p(z.DeviceBuffer.from_host(s)), z.sz(n), z._p(out), z._p(0))
    return out, out.to_host(np.uint32, (n, 36))


def normalised(dev, buf, n):
    return C.g1_normalise(buf.to_host(np.uint32, (n, 36)))


@pytest.mark.parametrize("m,n,bits", [(64, 3000, 14), (3, 40000, 14), (17, 1000, 31), (5, 300, 20), (1, 70000, 13)])
def test_commit_against_cpp_oracle(dev, m, n, bits):
    z = dev.z
    d_g, h_g = gpu_generators(dev, n, 1000 + n)
    rng = np.random.Generator(np.random.PCG64(m * n))
    sc = rng.integers(-(1 << bits), 1 << bits, size=m * n, dtype=np.int64).astype(np.int32)
    out = z.DeviceBuffer(144 * m)
    d_sc = z.DeviceBuffer.from_host(sc)
    dev.call("zkb_commit_i32", z._p(d_g), z.sz(n), z._p(d_sc), z.sz(m * n), z._p(out), z._p(0))
    exp = C.g1_normalise(C.commit_int(h_g, sc, "pippenger"))
    assert np.array_equal(normalised(dev, out, m), exp)
    for method in (1, 2):       # buckets, combination tables
        dev.call("zkb_memset0", z._p(out), z.sz(144 * m), z._p(0))
        dev.call("zkb_commit_i32_method", z._p(d_g), z.sz(n), z._p(d_sc), z.sz(m * n), z._p(out), ctypes.c_int(method), z._p(0))
        assert np.array_equal(normalised(dev, out, m), exp), method


def test_commit_is_linear_in_the_scalars(dev):
    """commit(a + b) = commit(a) + commit(b), 512 rows x 11008 generators (benchmark row length)"""
    z = dev.z
    m, n = 512, 11008
    d_g, _ = gpu_generators(dev, n, 7)
    rng = np.random.Generator(np.random.PCG64(99))
    a = np.rint(rng.standard_normal(m * n) * 0.02 * 65536).astype(np.int32)
    b = np.rint(rng.standard_normal(m * n) * 0.02 * 65536).astype(np.int32)
    outs = []
    for s in (a, b, a + b):
        o = z.DeviceBuffer(144 * m)
        dev.call("zkb_commit_i32", z._p(d_g), z.sz(n), z._p(z.DeviceBuffer.from_host(s)), z.sz(m * n), z._p(o), z._p(0))
        outs.append(o)
    summed = z.DeviceBuffer(144 * m)
    dev.call("zkb_g1_add", z._p(outs[0]), z._p(outs[1]), z._p(summed), z.sz(m), z._p(0))
    assert np.array_equal(normalised(dev, summed, m), normalised(dev, outs[2], m))
    # both algorithms give the same 512 points
    d_a = z.DeviceBuffer.from_host(a)
    by_method = []
    for method in (1, 2):
        o = z.DeviceBuffer(144 * m)
        dev.call("zkb_commit_i32_method", z._p(d_g), z.sz(n), z._p(d_a), z.sz(m * n), z._p(o), ctypes.c_int(method), z._p(0))
        by_method.append(normalised(dev, o, m))
    assert np.array_equal(by_method[0], by_method[1]) and np.array_equal(by_method[0], normalised(dev, outs[0], m))
    # and a sample of rows against the oracle
    _, h_g = gpu_generators(dev, n, 7)
    rows = [0, 255, 511]
    exp = C.commit_int(h_g, a.reshape(m, n)[rows], "pippenger")
    assert np.array_equal(normalised(dev, outs[0], m)[rows], C.g1_normalise(exp))


def _rand_fr(rng, k):
    v = rng.integers(0, 1 << 32, size=(max(k, 1), 8), dtype=np.uint64).astype(np.uint32)
    v[:, 7] %= np.uint32(R.R_MOD >> 224)
    return v[:k] if k else np.zeros((0, 8), dtype=np.uint32)


@pytest.mark.parametrize("B,I,O", [(64, 512, 768), (100, 300, 1000), (2048, 64, 128)])
def test_zkfc_against_cpp_oracle(dev, B, I, O):
    z = dev.z
    rng = np.random.Generator(np.random.PCG64(B + I + O))
    X = rng.integers(-70000, 70000, size=(B, I), dtype=np.int64)
    W = rng.integers(-5000, 5000, size=(I, O), dtype=np.int64)
    Y = X @ W
    fr = lambda a: R.fr_pack([int(v) for v in a.reshape(-1)])
    hX, hW, hY = fr(X), fr(W), fr(Y)
    ub, ui, uo = _rand_fr(rng, R.ceil_log2(B)), _rand_fr(rng, R.ceil_log2(I)), _rand_fr(rng, R.ceil_log2(O))
    rc, epolys, eclaims = C.zkfc_prove(hX, hW, hY, B, I, O, ub, ui, uo)
    assert rc == 0
    kI = ui.shape[0]
    polys = np.zeros((max(3 * kI, 1), 8), dtype=np.uint32)
    claims = np.zeros((4, 8), dtype=np.uint32)
    dev.call("zkb_zkfc_prove", z._p(z.fr_buffer(hX)), z._p(z.fr_buffer(hW)), z._p(z.fr_buffer(hY)), z.sz(B), z.sz(I), z.sz(O),
             z._p(z.fr_host(ub)), z._p(z.fr_host(ui)), z._p(z.fr_host(uo)), z._p(polys), z._p(claims), z._p(0))
    assert np.array_equal(polys[:3 * kI], epolys) and np.array_equal(claims, eclaims)
    # forward pass
    dY = z.DeviceBuffer(32 * B * O)
    dev.call("zkb_fr_matmul", z._p(z.fr_buffer(hX)), z._p(z.fr_buffer(hW)), z._p(dY), z.sz(B), z.sz(I), z.sz(O), z._p(0))
    assert np.array_equal(dY.to_host(np.uint32, (B * O, 8)), hY)


@pytest.mark.parametrize("logD,logN", [(16, 10), (18, 16), (14, 14)])
def test_tlookup_against_cpp_oracle(dev, logD, logN):
    z = dev.z
    D, N, low = 1 << logD, 1 << logN, -(1 << (logN - 1))
    rng = np.random.Generator(np.random.PCG64(logD * 100 + logN))
    S_int = rng.integers(low, low + N, size=D, dtype=np.int64).astype(np.int32)
    dS = z.DeviceBuffer(32 * D)
    dev.call("zkb_fr_from_i32", z._p(z.DeviceBuffer.from_host(S_int)), z._p(dS), z.sz(D), z._p(0))
    dT, dI, dM = z.DeviceBuffer(32 * N), z.DeviceBuffer(4 * D), z.DeviceBuffer(32 * N)
    dev.call("zkb_tlookup_range_table", z.i32(low), z.sz(N), z.sz(N), z._p(dT), z._p(0))
    dev.call("zkb_tlookup_range_indices", z._p(dS), z.i32(low), z._p(dI), z.sz(D), z._p(0))
    dev.call("zkb_tlookup_prep", z._p(dI), z.sz(D), z.sz(N), z._p(dM), z._p(0))
    hS, hT, hM = dS.to_host(np.uint32, (D, 8)), dT.to_host(np.uint32, (N, 8)), dM.to_host(np.uint32, (N, 8))
    assert np.array_equal(hM[:, 0], np.bincount(S_int.astype(np.int64) - low, minlength=N).astype(np.uint32))
    alpha, beta, u, v = _rand_fr(rng, 1), _rand_fr(rng, 1), _rand_fr(rng, logD), _rand_fr(rng, logD)
    rc, epolys, efinal = C.tlookup_prove(hS, hT, hM, alpha, beta, u, v)
    assert rc == 0
    polys = np.zeros((4 * logD, 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_tlookup_prove", z._p(dS), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u), z._p(v),
             z._p(polys), z._p(final), z._p(0))
    assert np.array_equal(polys, epolys) and np.array_equal(final, efinal)
    # table positions given: the inverses come from the table's, same transcript
    polys2, final2 = np.zeros_like(polys), np.zeros_like(final)
    dev.call("zkb_tlookup_prove_indexed", z._p(dS), z._p(dI), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u),
             z._p(v), z._p(polys2), z._p(final2), z._p(0))
    assert np.array_equal(polys2, epolys) and np.array_equal(final2, efinal)


def test_tlookup_full_size_verifies(dev):
    """2^23 lookups in a 2^16 table (the lookup benchmark size): all 23 round checks pass"""
    z = dev.z
    D, N, low = 1 << 23, 1 << 16, -(1 << 15)
    rng = np.random.Generator(np.random.PCG64(5))
    S_int = rng.integers(low, low + N, size=D, dtype=np.int64).astype(np.int32)
    dS = z.DeviceBuffer(32 * D)
    dev.call("zkb_fr_from_i32", z._p(z.DeviceBuffer.from_host(S_int)), z._p(dS), z.sz(D), z._p(0))
    dT, dI, dM = z.DeviceBuffer(32 * N), z.DeviceBuffer(4 * D), z.DeviceBuffer(32 * N)
    dev.call("zkb_tlookup_range_table", z.i32(low), z.sz(N), z.sz(N), z._p(dT), z._p(0))
    dev.call("zkb_tlookup_range_indices", z._p(dS), z.i32(low), z._p(dI), z.sz(D), z._p(0))
    dev.call("zkb_tlookup_prep", z._p(dI), z.sz(D), z.sz(N), z._p(dM), z._p(0))
    alpha, beta, u, v = _rand_fr(rng, 1), _rand_fr(rng, 1), _rand_fr(rng, 23), _rand_fr(rng, 23)
    polys = np.zeros((4 * 23, 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_tlookup_prove", z._p(dS), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u), z._p(v),
             z._p(polys), z._p(final), z._p(0))
    # a corrupted multiplicity must be caught
    bad = dM.to_host(np.uint32, (N, 8))
    bad[3, 0] += 1
    with pytest.raises(z.ZkbError) as e:
        dev.call("zkb_tlookup_prove", z._p(dS), z._p(dT), z._p(z.DeviceBuffer.from_host(bad)), z.sz(D), z.sz(N), z._p(alpha),
                 z._p(beta), z._p(u), z._p(v), z._p(polys), z._p(final), z._p(0))
    assert e.value.code == z.ERR_VERIFY


def _fr_of_ints(a):
    import bench
    return bench.ints_to_fr_limbs(np.asarray(a, dtype=np.int64))


@pytest.mark.parametrize("M,N,P,amax,bmax", [(128, 256, 128, 1 << 20, 3000), (100, 300, 150, (1 << 31) - 1, (1 << 31) - 1),
                                             (257, 129, 131, 70000, 70000), (64, 1024, 64, 1 << 31, 1 << 31),
                                             (128, 256, 128, 1 << 40, 3000), (100, 2048, 96, 1 << 60, 1 << 10),
                                             (64, 1024, 64, 1 << 60, 1 << 25), (70, 1000, 66, (1 << 62) + 5, 100)])
def test_matmul_integer_path_and_its_fallbacks(dev, M, N, P, amax, bmax):
    """large products of int32-encodings take the exact int64 kernel; a left operand beyond int32 (up to 2^61) is split
    into two 31-bit halves; products whose sums could pass 2^62 and operands that are not small integers take the field
    kernel; all agree with exact integer arithmetic"""
    z = dev.z
    rng = np.random.Generator(np.random.PCG64(M * N + P))
    A = rng.integers(-amax, amax, size=(M, N), dtype=np.int64)
    B = rng.integers(-bmax, bmax, size=(N, P), dtype=np.int64)
    A[0, 0], B[0, 0] = -amax, -bmax                       # includes -2^31 in the last case
    exp = [int(v) % R.R_MOD for v in (A.astype(object) @ B.astype(object)).reshape(-1)]
    dC = z.DeviceBuffer(32 * M * P)
    dev.call("zkb_fr_matmul", z._p(z.fr_buffer(_fr_of_ints(A))), z._p(z.fr_buffer(_fr_of_ints(B))), z._p(dC), z.sz(M), z.sz(N),
             z.sz(P), z._p(0))
    assert R.fr_unpack(dC.to_host(np.uint32, (M * P, 8))) == exp


@pytest.mark.parametrize("M,N,P,amax,bmax", [(300, 1000, 500, (1 << 23) - 1, (1 << 15) - 1), (257, 4100, 131, (1 << 23) - 1, (1 << 15) - 1),
                                             (129, 16384, 65, (1 << 23) - 1, (1 << 15) - 1), (512, 600, 512, 255, 255),
                                             (300, 1000, 500, 1 << 23, (1 << 15) - 1)])
def test_matmul_through_8_bit_limbs_on_the_tensor_cores(dev, M, N, P, amax, bmax):
    """left operand below 2^23, right operand below 2^15, at least 2^27 products: three and two byte limbs, six 8-bit
    tensor-core products with 32-bit accumulators, recombined exactly; extreme entries of both signs, ragged edges, the
    longest inner dimension the accumulators allow; the last case is one past the limb range and takes the int64 kernel"""
    z = dev.z
    rng = np.random.Generator(np.random.PCG64(M + N + P))
    A = rng.integers(-amax, amax + 1, size=(M, N), dtype=np.int64)
    B = rng.integers(-bmax, bmax + 1, size=(N, P), dtype=np.int64)
    A[0, :], B[:, 0] = amax, bmax                         # the largest sums of products, both signs
    A[1, :], B[:, 1] = -amax, bmax
    A[2, :], B[:, 2] = -amax, -bmax
    exp = [int(v) % R.R_MOD for v in (A @ B).reshape(-1)]  # exact in int64: |sum| < 2^23 2^15 2^14
    dC = z.DeviceBuffer(32 * M * P)
    dev.call("zkb_fr_matmul", z._p(z.fr_buffer(_fr_of_ints(A))), z._p(z.fr_buffer(_fr_of_ints(B))), z._p(dC), z.sz(M), z.sz(N),
             z.sz(P), z._p(0))
    assert R.fr_unpack(dC.to_host(np.uint32, (M * P, 8))) == exp


def test_matmul_with_general_field_elements_uses_the_field_kernel(dev):
    z = dev.z
    M, N, P = 96, 512, 96
    rng = np.random.Generator(np.random.PCG64(3))
    A = rng.integers(-1000, 1000, size=(M, N), dtype=np.int64)
    hA = _fr_of_ints(A)
    hB = _rand_fr(rng, N * P)
    dC = z.DeviceBuffer(32 * M * P)
    dev.call("zkb_fr_matmul", z._p(z.fr_buffer(hA)), z._p(z.fr_buffer(hB)), z._p(dC), z.sz(M), z.sz(N), z.sz(P), z._p(0))
    Bv = R.fr_unpack(hB)
    got = R.fr_unpack(dC.to_host(np.uint32, (M * P, 8)))
    for (i, j) in ((0, 0), (5, 7), (95, 95), (40, 3)):
        assert got[i * P + j] == sum(int(A[i, k]) * Bv[k * P + j] for k in range(N)) % R.R_MOD


def _rand_fr_limbs(rng, n):
    s = rng.integers(0, 1 << 32, size=(n, 8), dtype=np.uint64).astype(np.uint32)
    s[:, 7] %= np.uint32(R.R_MOD >> 224)
    return s


def _me_open(dev, d_t, d_g, n, u):
    z = dev.z
    k = u.shape[0]
    hp = np.zeros((3 * k + 1, 36), dtype=np.uint32)
    ho = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_me_open", z._p(d_t), z._p(d_g), z.sz(n), z._p(u if k else np.zeros((1, 8), np.uint32)), z.u32(k), z._p(hp),
             z._p(ho), z._p(0))
    return hp, ho


@pytest.mark.parametrize("n,k", [(300, 9), (1000, 10), (4096, 12), (4097, 13)])
def test_me_open_against_cpp_oracle(dev, n, k):
    """opening proof with odd lengths along the way (300 -> 150 -> 75 -> 38 -> 19 ...) and several column segments"""
    z = dev.z
    d_g, h_g = gpu_generators(dev, n, 31 + n)
    rng = np.random.Generator(np.random.PCG64(n + k))
    t, u = _rand_fr_limbs(rng, n), _rand_fr_limbs(rng, k)
    hp, ho = _me_open(dev, z.DeviceBuffer.from_host(t), d_g, n, u)
    exp_proof, exp_out = C.me_open(t, h_g, u)
    assert np.array_equal(ho, exp_out)
    assert np.array_equal(C.g1_normalise(hp), C.g1_normalise(exp_proof))


def test_openings_in_flight_equal_the_blocking_call(dev):
    """zkb_me_open_begin / zkb_me_open_end: five openings of different sizes started back to back (four run side by side on
    streams of their own, the fifth finds every lane taken and runs inside begin), other work queued meanwhile, then collected
    in another order; proof elements and openings equal zkb_me_open's."""
    import ctypes
    z = dev.z
    rng = np.random.Generator(np.random.PCG64(77))
    cases = []
    for n, k in ((5000, 13), (300, 9), (4096, 12), (9000, 14), (1, 0)):
        d_g, _ = gpu_generators(dev, n, 500 + n)
        t = _rand_fr_limbs(rng, n)
        d_t = z.DeviceBuffer.from_host(t)
        u = _rand_fr_limbs(rng, max(k, 1))
        want = _me_open(dev, d_t, d_g, n, u[:k])
        cases.append((n, k, d_g, d_t, u, want))
    handles = []
    for n, k, d_g, d_t, u, _ in cases:
        h = ctypes.c_void_p()
        dev.call("zkb_me_open_begin", z._p(d_t), z._p(d_g), z.sz(n), z._p(u), z.u32(k), z._p(0), ctypes.byref(h))
        handles.append(h)
    # something else on the default stream while they run
    a = z.DeviceBuffer.from_host(_rand_fr_limbs(rng, 1 << 16))
    dev.call("zkb_fr_mul", z._p(a), z._p(a), z._p(a), z.sz(1 << 16), z._p(0))
    for i in (2, 0, 4, 1, 3):
        n, k, d_g, d_t, u, (want_p, want_o) = cases[i]
        hp, ho = np.zeros((3 * k + 1, 36), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        dev.call("zkb_me_open_end", handles[i], z._p(hp), z._p(ho))
        assert np.array_equal(ho, want_o)
        assert np.array_equal(C.g1_normalise(hp), C.g1_normalise(want_p))


def test_me_open_with_identity_generators_and_zero_scalars(dev):
    z = dev.z
    n, k = 600, 10
    d_g, h_g = gpu_generators(dev, n, 5)
    h_g = h_g.copy()
    h_g[[0, 7, 8, 9, 599]] = 0                      # Z = 0: the identity
    h_g[11] = h_g[10]                               # equal neighbours: g0 - g1 is the identity
    d_g = z.DeviceBuffer.from_host(h_g)
    rng = np.random.Generator(np.random.PCG64(77))
    t, u = _rand_fr_limbs(rng, n), _rand_fr_limbs(rng, k)
    t[[3, 4, 8, 100]] = 0
    u[2] = 0
    u[3] = R.fr_pack([1])[0]
    hp, ho = _me_open(dev, z.DeviceBuffer.from_host(t), d_g, n, u)
    exp_proof, exp_out = C.me_open(t, h_g, u)
    assert np.array_equal(ho, exp_out)
    assert np.array_equal(C.g1_normalise(hp), C.g1_normalise(exp_proof))


@pytest.mark.parametrize("n", [100000, 1 << 19])
def test_me_open_round_identities_at_full_width(dev, n):
    """Size-independent check of an opening over 2^19 generators (the FFN weights' row length): with
    s' = s0 + u (s1 - s0) and g' = g1 + u (g0 - g1), the next round's T is u(1-u) T + (1-u)^2 T0 + u^2 T1, the last one is
    (final scalar) * (final generator), and the first T is the plain sum of products."""
    z = dev.z
    k = (n - 1).bit_length()
    d_g, _ = gpu_generators(dev, n, 2024)
    rng = np.random.Generator(np.random.PCG64(n))
    t, u = _rand_fr_limbs(rng, n), _rand_fr_limbs(rng, k)
    d_t = z.DeviceBuffer.from_host(t)
    hp, ho = _me_open(dev, d_t, d_g, n, u)
    # first T by the elementwise product kernel and the tree sum
    prod = z.DeviceBuffer(144 * n)
    dev.call("zkb_g1_mul", z._p(d_g), z.sz(n), z._p(d_t), z.sz(n), z._p(prod), z._p(0))
    t0 = np.zeros((1, 36), dtype=np.uint32)
    dev.call("zkb_g1_sum", z._p(prod), z.sz(n), z._p(t0), z._p(0))
    assert np.array_equal(C.g1_normalise(t0), C.g1_normalise(np.ascontiguousarray(hp[0:1])))
    uu = R.fr_unpack(u)
    coeff = []
    for x in uu:
        coeff += [x * (1 - x) % R.R_MOD, (1 - x) * (1 - x) % R.R_MOD, x * x % R.R_MOD]
    terms = C.g1_mul(np.ascontiguousarray(hp[:3 * k]), R.fr_pack(coeff))
    part = [np.ascontiguousarray(terms[i::3]) for i in range(3)]
    nxt = C.g1_add(C.g1_add(part[0], part[1]), part[2])          # T of round r + 1, for r = 0..k-1
    last = C.g1_mul(np.ascontiguousarray(hp[3 * k:3 * k + 1]), ho)                                  # final scalar (raw limbs) * final generator
    expect = np.ascontiguousarray(np.concatenate([hp[3:3 * k:3], last]))
    assert np.array_equal(C.g1_normalise(nxt), C.g1_normalise(expect))


def test_block_evaluations_combine_like_the_sharded_path(dev):
    """The multi-GPU split of a multilinear evaluation, with the ranks emulated in one process: each block of a 2^20-element
    tensor is evaluated on the device at the low challenges, the blocks are weighted by eq(high challenges; rank) as
    sharding.sharded_mle_combine does, and the sum equals the device evaluation of the whole tensor."""
    from zkllm_ccs2024_b200 import sharding as S
    z = dev.z
    k, kw = 20, 2                                   # 4 ranks
    rng = np.random.Generator(np.random.PCG64(5))
    t = _rand_fr_limbs(rng, 1 << k)
    u = _rand_fr_limbs(rng, k)
    d_t = z.DeviceBuffer.from_host(t)
    whole = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_fr_mle_eval", z._p(d_t), z.sz(1 << k), z._p(u), z.u32(k), z._p(whole), z._p(0))
    u_high = S.fr_limbs_to_ints(u[k - kw:])
    acc = 0
    n_local = 1 << (k - kw)
    for rank in range(1 << kw):
        d_block = z.DeviceBuffer.from_host(np.ascontiguousarray(t[rank * n_local:(rank + 1) * n_local]))
        part = np.zeros((1, 8), dtype=np.uint32)
        dev.call("zkb_fr_mle_eval", z._p(d_block), z.sz(n_local), z._p(np.ascontiguousarray(u[:k - kw])), z.u32(k - kw), z._p(part),
                 z._p(0))
        acc = (acc + S.fr_limbs_to_ints(part)[0] * S.block_weight(u_high, rank)) % S.R_MOD
    assert acc == S.fr_limbs_to_ints(whole)[0]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_zkip_equals_the_whole_sumcheck(dev, world):
    """The multi-GPU split of zkip with the ranks emulated in one process: every rank's round-robin share runs its
    local rounds on the device (zkb_zkip_partial), sharding.zkip_combine adds the coefficient sums, runs the last
    log2(world) rounds on the surviving pairs and replays the verifier; polynomials and final claim equal zkb_zkip's."""
    from zkllm_ccs2024_b200 import sharding as S
    z = dev.z
    k = 16
    n = 1 << k
    rng = np.random.Generator(np.random.PCG64(world))
    a, b, u = _rand_fr_limbs(rng, n), _rand_fr_limbs(rng, n), _rand_fr_limbs(rng, k)
    ai, bi = S.fr_limbs_to_ints(a), S.fr_limbs_to_ints(b)
    claim = sum(x * y for x, y in zip(ai, bi)) % S.R_MOD
    polys = np.zeros((3 * k, 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_zkip", z._p(S.fr_ints_to_limbs([claim])), z._p(z.DeviceBuffer.from_host(a)), z._p(z.DeviceBuffer.from_host(b)), z.sz(n),
             z._p(u), z.u32(k), z._p(polys), z._p(final), z._p(0))
    rounds = S.zkip_local_rounds(n // world)
    per_rank = []
    for rank in range(world):
        la, lb = np.ascontiguousarray(a[rank::world]), np.ascontiguousarray(b[rank::world])
        sums = np.zeros((3 * rounds, 8), dtype=np.uint32)
        ta, tb = np.zeros((1, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        dev.call("zkb_zkip_partial", z._p(z.DeviceBuffer.from_host(la)), z._p(z.DeviceBuffer.from_host(lb)), z.sz(n // world), z._p(u),
                 z.u32(k), z.u32(rounds), z._p(sums), z._p(ta), z._p(tb), z._p(0))
        v = S.fr_limbs_to_ints(sums)
        per_rank.append(([v[3 * r:3 * r + 3] for r in range(rounds)], S.fr_limbs_to_ints(ta), S.fr_limbs_to_ints(tb)))
    got_polys, got_final = S.zkip_combine(per_rank, S.fr_limbs_to_ints(u), claim)
    want = S.fr_limbs_to_ints(polys)
    assert got_polys == [want[3 * r:3 * r + 3] for r in range(k)]
    assert got_final == S.fr_limbs_to_ints(final)[0]


@pytest.mark.parametrize("world", [2, 8])
def test_sharded_zkfc_prove_equals_the_single_gpu_proof(dev, world):
    """zkFC::prove's body with W dealt out by rows (and X by the matching columns) over `world` emulated ranks: the
    proof polynomials and the four claims equal what zkb_zkfc_prove returns for the whole tensors."""
    from zkllm_ccs2024_b200 import sharding as S
    z = dev.z
    B, I, O = 16, 512, 128
    rng = np.random.Generator(np.random.PCG64(40 + world))
    X = rng.integers(-3000, 3000, size=(B, I), dtype=np.int64)
    W = rng.integers(-3000, 3000, size=(I, O), dtype=np.int64)
    Y = X @ W
    ub, ui, uo = _rand_fr_limbs(rng, 4), _rand_fr_limbs(rng, 9), _rand_fr_limbs(rng, 7)
    dX, dW, dY = (z.fr_buffer(_fr_of_ints(t)) for t in (X, W, Y))
    polys = np.zeros((27, 8), dtype=np.uint32)
    claims = np.zeros((4, 8), dtype=np.uint32)
    dev.call("zkb_zkfc_prove", z._p(dX), z._p(dW), z._p(dY), z.sz(B), z.sz(I), z.sz(O), z._p(ub), z._p(ui), z._p(uo), z._p(polys),
             z._p(claims), z._p(0))
    parts = []
    for rank in range(world):
        dXl = z.fr_buffer(_fr_of_ints(np.ascontiguousarray(X[:, rank::world])))
        dWl = z.fr_buffer(_fr_of_ints(np.ascontiguousarray(W[rank::world, :])))
        parts.append(S.zkfc_local_part(z, dXl, dWl, B, I // world, O, ub, ui, uo, world))
    want_claims = S.fr_limbs_to_ints(claims)
    got = S.zkfc_combine(parts, want_claims[0], S.fr_limbs_to_ints(ui))
    want_polys = S.fr_limbs_to_ints(polys)
    assert got["proof"] == [want_polys[3 * r:3 * r + 3] for r in range(9)]
    assert [got["claim"], got["final_claim"], got["claim_x"], got["claim_w"]] == want_claims


def test_row_folds_of_mixed_tensors_match_the_field_matmul(dev):
    """FrTensor::partial_me along the last axis of a [2400, 3000] tensor (one warp per part of a row, lazily reduced
    small-integer products) against an independent path: the field matmul of the tensor with the eq table.  Entries mix
    small integers of both signs, 64-bit integers, zeros and arbitrary field elements."""
    z = dev.z
    rows, J, k = 2400, 3000, 12
    rng = np.random.Generator(np.random.PCG64(77))
    vals = rng.integers(-(1 << 20), 1 << 20, size=rows * J, dtype=np.int64)
    vals[::7] = rng.integers(-(1 << 62), 1 << 62, size=vals[::7].size, dtype=np.int64)
    vals[::11] = 0
    t = _fr_of_ints(vals)
    t[5::13] = _rand_fr_limbs(rng, t[5::13].shape[0])           # not small in either sign
    u = _rand_fr_limbs(rng, k)
    uu = R.fr_unpack(u)
    eq = [1]
    for x in uu:                                                 # index bit j pairs with challenge j
        eq = [e * (1 - x) % R.R_MOD for e in eq] + [e * x % R.R_MOD for e in eq]
    d_t = z.DeviceBuffer.from_host(t)
    got = z.DeviceBuffer(32 * rows)
    dev.call("zkb_fr_partial_me", z._p(d_t), z.sz(rows * J), z._p(u), z.u32(k), z.sz(J), z.sz(1), z._p(got), z._p(0))
    want = z.DeviceBuffer(32 * rows)
    dev.call("zkb_fr_matmul", z._p(d_t), z._p(z.fr_buffer(R.fr_pack(eq[:J]))), z._p(want), z.sz(rows), z.sz(J), z.sz(1), z._p(0))
    assert np.array_equal(got.to_host(np.uint32, (rows, 8)), want.to_host(np.uint32, (rows, 8)))
    # and two rows against exact integer arithmetic
    tv = R.fr_unpack(t[:2 * J])
    for r_ in range(2):
        assert R.fr_unpack(got.to_host(np.uint32, (rows, 8))[r_:r_ + 1])[0] == sum(a * e for a, e in zip(tv[r_ * J:(r_ + 1) * J], eq)) % R.R_MOD


def test_mle_eval_of_small_integers(dev):
    """the lazily reduced dot product inside the multilinear evaluation, on fixed-point values up to 64 bits"""
    z = dev.z
    n, k = 5000, 13
    rng = np.random.Generator(np.random.PCG64(78))
    vals = rng.integers(-(1 << 63), (1 << 63) - 1, size=n, dtype=np.int64)
    vals[:8] = [0, 1, -1, (1 << 32) - 1, 1 << 32, -(1 << 32), (1 << 63) - 1, -(1 << 63)]
    u = _rand_fr_limbs(rng, k)
    out = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_fr_mle_eval", z._p(z.fr_buffer(_fr_of_ints(vals))), z.sz(n), z._p(u), z.u32(k), z._p(out), z._p(0))
    assert R.fr_unpack(out)[0] == R.mle_eval([int(v) % R.R_MOD for v in vals], R.fr_unpack(u))


@pytest.mark.parametrize("world,logD,logN", [(2, 14, 8), (4, 16, 10), (8, 13, 13), (8, 18, 7)])
def test_sharded_tlookup_equals_the_whole_proof(dev, world, logD, logN):
    """The multi-GPU split of tLookup::prove with the ranks emulated in one process: values, table and multiplicities dealt
    out round-robin, every rank's local rounds on the device (zkb_tlookup_partial), sharding.tlookup_combine for the
    exchange, the shared last rounds and the replay; polynomials and final claim equal zkb_tlookup_prove's."""
    from zkllm_ccs2024_b200 import sharding as S
    z = dev.z
    D, N, low = 1 << logD, 1 << logN, -(1 << (logN - 1))
    rng = np.random.Generator(np.random.PCG64(world * 1000 + logD))
    S_int = rng.integers(low, low + N, size=D, dtype=np.int64).astype(np.int32)
    dS = z.DeviceBuffer(32 * D)
    dev.call("zkb_fr_from_i32", z._p(z.DeviceBuffer.from_host(S_int)), z._p(dS), z.sz(D), z._p(0))
    dT, dI, dM = z.DeviceBuffer(32 * N), z.DeviceBuffer(4 * D), z.DeviceBuffer(32 * N)
    dev.call("zkb_tlookup_range_table", z.i32(low), z.sz(N), z.sz(N), z._p(dT), z._p(0))
    dev.call("zkb_tlookup_range_indices", z._p(dS), z.i32(low), z._p(dI), z.sz(D), z._p(0))
    dev.call("zkb_tlookup_prep", z._p(dI), z.sz(D), z.sz(N), z._p(dM), z._p(0))
    hS, hT, hM = dS.to_host(np.uint32, (D, 8)), dT.to_host(np.uint32, (N, 8)), dM.to_host(np.uint32, (N, 8))
    alpha, beta, u, v = _rand_fr(rng, 1), _rand_fr(rng, 1), _rand_fr(rng, logD), _rand_fr(rng, logD)
    polys = np.zeros((4 * logD, 8), dtype=np.uint32)
    final = np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_tlookup_prove", z._p(dS), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u), z._p(v),
             z._p(polys), z._p(final), z._p(0))
    ui, vi = S.fr_limbs_to_ints(u), S.fr_limbs_to_ints(v)
    ul, vl = S.tlookup_local_challenges(ui, vi, D, N, world)
    rounds = logD - (world.bit_length() - 1)
    per_rank = []
    for rank in range(world):
        shares = [z.DeviceBuffer.from_host(np.ascontiguousarray(h[rank::world])) for h in (hS, hT, hM)]
        sums = np.zeros((1 + 11 * rounds, 8), dtype=np.uint32)
        tails = np.zeros((5, 8), dtype=np.uint32)
        dev.call("zkb_tlookup_partial", z._p(shares[0]), z._p(shares[1]), z._p(shares[2]), z.sz(D // world), z.sz(N // world), z._p(beta),
                 z._p(S.fr_host_or_dummy(S.fr_ints_to_limbs(ul))), z._p(S.fr_host_or_dummy(S.fr_ints_to_limbs(vl))), z.u32(rounds),
                 z._p(sums), z._p(tails), z._p(0))
        t = S.fr_limbs_to_ints(tails)
        per_rank.append((S.fr_limbs_to_ints(sums), [t[0]], [t[1]], [t[2]], [t[3]], [t[4]]))
    got_polys, got_final = S.tlookup_combine(per_rank, D, N, S.fr_limbs_to_ints(alpha)[0], S.fr_limbs_to_ints(beta)[0], ui, vi)
    want = S.fr_limbs_to_ints(polys)
    assert got_polys == [want[4 * r:4 * r + 4] for r in range(logD)]
    assert got_final == S.fr_limbs_to_ints(final)[0]
    # the C++ twin of the combine on the same gathered blocks
    flat = []
    for sums_p, a_, s_, b_, t_, m_ in per_rank:
        flat += sums_p + a_ + s_ + b_ + t_ + m_
    cpolys, cfinal = np.zeros((4 * logD, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    dev.call("zkb_tlookup_combine", z._p(S.fr_ints_to_limbs(flat)), z.u32(world), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u),
             z._p(v), z._p(cpolys), z._p(cfinal))
    assert np.array_equal(cpolys, polys) and np.array_equal(cfinal, final)


@pytest.mark.parametrize("world,K,logN", [(2, 3, 12), (4, 2, 14), (8, 4, 10), (8, 2, 3)])
def test_sharded_multi_hadamard_equals_the_whole_proof(dev, world, K, logN):
    """The multi-GPU split of multi_hadamard_sumchecks with the ranks emulated in one process: every rank's rounds on the
    device (zkb_multi_hadamard_partial on its round-robin share), then zkb_multi_hadamard_combine and its Python twin;
    polynomials and final claim equal zkb_multi_hadamard's on the whole tensors."""
    import ctypes
    from zkllm_ccs2024_b200 import sharding as S
    z = dev.z
    N = 1 << logN
    kP = world.bit_length() - 1
    rng = np.random.Generator(np.random.PCG64(world * 100 + K * 10 + logN))
    Xs = [_rand_fr(rng, N) for _ in range(K)]
    u, v = _rand_fr(rng, logN), _rand_fr(rng, logN)
    bufs = [z.fr_buffer(x) for x in Xs]
    prod, claim = z.DeviceBuffer(32 * N), np.zeros((1, 8), dtype=np.uint32)
    first = bufs[0]
    for j in range(1, K):
        dev.call("zkb_fr_mul", z._p(first), z._p(bufs[j]), z._p(prod), z.sz(N), z._p(0))
        first = prod
    dev.call("zkb_fr_mle_eval", z._p(first), z.sz(N), z._p(u), z.u32(logN), z._p(claim), z._p(0))
    polys, final = np.zeros((logN * (K + 1), 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    ptrs = (ctypes.c_void_p * K)(*[b.ptr for b in bufs])
    dev.call("zkb_multi_hadamard", z._p(claim), ptrs, z.u32(K), z.sz(N), z._p(u), z._p(v), z._p(polys), z._p(final), z._p(0))
    local = logN - kP
    block = local * (K + 1) + K
    parts = np.zeros((world, block, 8), dtype=np.uint32)
    for rank in range(world):
        shares = [z.fr_buffer(np.ascontiguousarray(x[rank::world])) for x in Xs]
        sp = (ctypes.c_void_p * K)(*[b.ptr for b in shares])
        dev.call("zkb_multi_hadamard_partial", sp, z.u32(K), z.sz(N // world), z._p(S.fr_host_or_dummy(u[kP:])),
                 z._p(S.fr_host_or_dummy(v[kP:])), z._p(parts[rank]), z._p(parts[rank, local * (K + 1):]), z._p(0))
    cpolys, cfinal = np.zeros_like(polys), np.zeros_like(final)
    dev.call("zkb_multi_hadamard_combine", z._p(parts), z.u32(world), z.u32(K), z.u32(logN), z._p(u), z._p(v), z._p(claim), z._p(cpolys),
             z._p(cfinal))
    assert np.array_equal(cpolys, polys) and np.array_equal(cfinal, final)
    per_rank = []
    for rank in range(world):
        vals = S.fr_limbs_to_ints(parts[rank])
        per_rank.append(([vals[r * (K + 1):(r + 1) * (K + 1)] for r in range(local)], vals[local * (K + 1):]))
    got_polys, got_final = S.multi_hadamard_combine(per_rank, S.fr_limbs_to_ints(u), S.fr_limbs_to_ints(v), S.fr_limbs_to_ints(claim)[0])
    want = S.fr_limbs_to_ints(polys)
    assert got_polys == [want[r * (K + 1):(r + 1) * (K + 1)] for r in range(logN)]
    assert got_final == S.fr_limbs_to_ints(final)[0]


def test_host_buffer_commitment_equals_the_device_path(dev):
    """zkb_commit_i32_host on a 1030 x 16384 matrix with 31-bit entries in some rows (five windows) against
    zkb_commit_i32 on device buffers, and three rows against the C++ oracle."""
    z = dev.z
    m, n = 1030, 16384
    d_g, h_g = gpu_generators(dev, n, 4242)
    rng = np.random.Generator(np.random.PCG64(31))
    sc = rng.integers(-8000, 8000, size=(m, n), dtype=np.int64).astype(np.int32)
    sc[300:520] = rng.integers(-(1 << 30), 1 << 30, size=(220, n), dtype=np.int64).astype(np.int32)
    sc[m - 1] = 0
    h_out = np.zeros((m, 36), dtype=np.uint32)
    dev.call("zkb_commit_i32_host", z._p(h_g), z.sz(n), z._p(sc.reshape(-1)), z.sz(m * n), z._p(h_out), z._p(0))
    d_out = z.DeviceBuffer(144 * m)
    dev.call("zkb_commit_i32", z._p(d_g), z.sz(n), z._p(z.DeviceBuffer.from_host(sc.reshape(-1))), z.sz(m * n), z._p(d_out), z._p(0))
    assert np.array_equal(C.g1_normalise(h_out), normalised(dev, d_out, m))
    rows = [0, 400, m - 1]
    exp = C.commit_int(h_g, np.ascontiguousarray(sc[rows]).reshape(-1), "pippenger")
    assert np.array_equal(C.g1_normalise(np.ascontiguousarray(h_out[rows])), C.g1_normalise(exp))
