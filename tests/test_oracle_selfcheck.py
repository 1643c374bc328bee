"""CPU: the big-integer oracle against the verifier identities the reference
asserts at its throw sites, and against algebraic facts that do not depend on it."""
import random

import pytest

from oracle import pyref as R
from tests.util import rand_fr, rand_small_fr, seeded_generators


def test_constants():
    assert R.FR_RADIX == pow(2, 256, R.R_MOD) and R.FQ_RADIX == pow(2, 384, R.Q_MOD)
    assert (R.G1_Y ** 2 - R.G1_X ** 3 - 4) % R.Q_MOD == 0
    assert R.TWO_INV * 2 % R.R_MOD == 1
    # the reference's TWO_INV literal (tlookup.cu:180)
    lit = [2147483649, 2147483647, 2147429887, 2849952257, 80800770, 429714436, 2496577188, 972477353]
    assert R.limbs_to_int(lit) == R.TWO_INV
    # G1 generator in Montgomery form (g1-tensor.cuh:29-58), first and last limbs
    gx = R.G1_X * R.FQ_RADIX % R.Q_MOD
    assert gx & 0xFFFFFFFF == 4250078230 and gx >> (32 * 11) == 302085953
    assert R.g1_affine(R.g1_mul(R.G1_GEN, R.R_MOD)) is None          # group order


def test_mle_is_multilinear_extension():
    rng = random.Random(0)
    for n in (1, 2, 3, 5, 8, 13):
        k = R.ceil_log2(n)
        t = rand_fr(rng, n)
        for idx in range(1 << k):
            u = [(idx >> j) & 1 for j in range(k)]
            assert R.mle_eval(t, u) == (t[idx] if idx < n else 0)


def test_partial_me_matches_full_eval():
    rng = random.Random(1)
    d0, d1 = 5, 7
    t = rand_fr(rng, d0 * d1)
    u0, u1 = rand_fr(rng, 3), rand_fr(rng, 3)
    rows = R.partial_me(t, u1, d1, 1)
    assert R.mle_eval(rows, u0) == R.multi_dim_me(t, [u0, u1], [d0, d1])
    cols = R.partial_me(t, u0, d0, d1)
    assert R.mle_eval(cols, u1) == R.multi_dim_me(t, [u0, u1], [d0, d1])
    # padding an axis to a power of two does not change the evaluation
    assert R.mle_eval(R.pad(t, [d0, d1]), u1 + u0) == R.multi_dim_me(t, [u0, u1], [d0, d1])


@pytest.mark.parametrize("B,I,O", [(1, 1, 4), (2, 4, 4), (3, 5, 7), (4, 1, 6)])
def test_zkfc_prove_identities(B, I, O):
    rng = random.Random(B * 100 + I * 10 + O)
    X, W = rand_small_fr(rng, B * I), rand_small_fr(rng, I * O)
    Y = R.matmul(X, W, B, I, O)
    out = R.zkfc_prove(X, W, Y, B, I, O, rand_fr(rng, R.ceil_log2(B)), rand_fr(rng, R.ceil_log2(I)), rand_fr(rng, R.ceil_log2(O)))
    assert out["final_claim"] == out["claim_x"] * out["claim_w"] % R.R_MOD
    Y[0] = (Y[0] + 1) % R.R_MOD
    with pytest.raises(RuntimeError):
        R.zkfc_prove(X, W, Y, B, I, O, rand_fr(rng, R.ceil_log2(B)), rand_fr(rng, R.ceil_log2(I)), rand_fr(rng, R.ceil_log2(O)))


@pytest.mark.parametrize("D,N", [(4, 4), (16, 4), (64, 8), (8, 1)])
def test_tlookup_identities(D, N):
    rng = random.Random(D + N)
    low = -3
    table = R.range_table(low, N)
    vals = [R.int_to_fr(rng.randrange(low, low + N)) for _ in range(D)]
    m = R.tlookup_prep(R.range_indices(vals, low), N)
    k = R.ceil_log2(D)
    polys = []
    R.tlookup_prove(vals, table, m, rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rand_fr(rng, k), rand_fr(rng, k), polys)
    assert len(polys) == k
    bad = list(m)
    bad[0] = (bad[0] + 1) % R.R_MOD
    with pytest.raises(RuntimeError):
        R.tlookup_prove(vals, table, bad, rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rand_fr(rng, k), rand_fr(rng, k))


def test_mapping_lookup_pads_non_power_of_two():
    rng = random.Random(4)
    low, N = 0, 8
    table = R.range_table(low, N)
    mapped = rand_fr(rng, N)
    D = 12
    s_in = [R.int_to_fr(rng.randrange(low, low + N)) for _ in range(D)]
    idx = R.range_indices(s_in, low)
    s_out = [mapped[i] for i in idx]
    m = R.tlookup_prep(idx, N)
    k = 4
    R.tlookup_mapping_prove(s_in, s_out, table, mapped, m, rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rng.randrange(R.R_MOD),
                            rand_fr(rng, k), rand_fr(rng, k))


def test_multi_hadamard_identity():
    rng = random.Random(5)
    for K, N in ((1, 4), (2, 8), (3, 16)):
        Xs = [rand_fr(rng, N) for _ in range(K)]
        k = R.ceil_log2(N)
        u, v = rand_fr(rng, k), rand_fr(rng, k)
        prod = [1] * N
        for X in Xs:
            prod = [p * x % R.R_MOD for p, x in zip(prod, X)]
        out = R.multi_hadamard_sumchecks(R.mle_eval(prod, u), Xs, u, v, [])
        exp = 1
        for X in Xs:
            # MSB-first folds with v consumed from the back = LSB-first evaluation at v
            exp = exp * R.mle_eval(X, v) % R.R_MOD
        assert out == exp


def test_commit_and_open_are_consistent():
    rng = random.Random(6)
    gens = seeded_generators(4, 42)
    rows = 2
    t_int = [rng.randrange(-100, 100) for _ in range(rows * 4)]
    t = [R.int_to_fr(v) for v in t_int]
    com = R.commit_int(gens, t)
    full = R.commit(gens, t)
    for a, b in zip(com, full):
        assert R.g1_affine(a) == R.g1_affine(b)
    u = rand_fr(rng, 3)
    proof = []
    opening = R.commitment_open(gens, t, rows, u, proof)
    assert opening == R.mle_eval(t, u)          # the opening is the MLE of the committed tensor
    assert len(proof) == 3 * 2 + 1
    # first round element = commitment of the row-folded tensor under the generators
    folded = R._legacy_partial_me(t, u[2:], 4)
    assert R.g1_affine(proof[0]) == R.g1_affine(R.commit(gens, folded)[0])


def test_rescale_identity_and_legacy_factor():
    rng = random.Random(7)
    x = [R.int_to_fr(rng.randrange(-2**40, 2**40)) for _ in range(100)]
    out, rem = R.rescale(x, 1 << 16)
    for a, o, r_ in zip(x, out, rem):
        assert R.fr_to_long(o) * 65536 + R.fr_to_long(r_) == R.fr_to_long(a)
        assert -32768 <= R.fr_to_long(r_) < 32768
    a, b = rand_fr(rng, 8), rand_fr(rng, 8)
    u = rand_fr(rng, 3)
    pr = R.inner_product_sumcheck(a, b, u)
    # round 0: p(0) + p(1) = <a, b> / R  (the reference leaves the Montgomery factor in)
    ip = sum(x_ * y_ for x_, y_ in zip(a, b)) % R.R_MOD
    assert (2 * pr[0] + pr[1] + pr[2]) % R.R_MOD == ip * R.FR_RADIX_INV % R.R_MOD
