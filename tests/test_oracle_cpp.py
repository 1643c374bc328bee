"""CPU: the C++ restatement (oracle/zkoracle.cpp) against the Python big-integer oracle."""
import random

import numpy as np

from oracle import cpporacle as C
from oracle import pyref as R
from tests.util import EDGE_FR, rand_fr, rand_small_fr, seeded_generators


def test_field_ops():
    rng = random.Random(0)
    a = EDGE_FR + rand_fr(rng, 200)
    b = list(reversed(EDGE_FR)) + rand_fr(rng, 200)
    assert R.fr_unpack(C.fr_mul(R.fr_pack(a), R.fr_pack(b))) == [x * y % R.R_MOD for x, y in zip(a, b)]
    assert R.fr_unpack(C.fr_inv(R.fr_pack(a[:40]))) == [R.fr_inv(x) for x in a[:40]]


def test_group_ops_and_commit():
    rng = random.Random(1)
    gens = seeded_generators(12, 7)
    a, b = gens[:6] + [R.G1_ZERO, gens[0], gens[1]], gens[6:] + [gens[2], gens[0], R.g1_neg(gens[1])]
    out = R.g1_unpack(C.g1_add(R.g1_pack(a), R.g1_pack(b)))
    for x, y, z in zip(a, b, out):
        assert R.g1_affine(z) == R.g1_affine(R.g1_add(x, y))
    ks = rand_fr(rng, 4)
    out = R.g1_unpack(C.g1_mul(R.g1_pack(gens[:4]), R.fr_pack(ks)))
    for g, k, z in zip(gens, ks, out):
        assert R.g1_affine(z) == R.g1_affine(R.g1_mul(g, k))
    ints = np.array([rng.randrange(-9000, 9000) for _ in range(3 * 12)] , dtype=np.int32)
    ints[0], ints[1], ints[2] = 0, -(1 << 31), (1 << 31) - 1
    exp = R.commit_int(gens, [R.int_to_fr(int(v)) for v in ints])
    for algo in ("ref", "pippenger"):
        out = R.g1_unpack(C.commit_int(R.g1_pack(gens), ints, algo))
        for z, e in zip(out, exp):
            assert R.g1_affine(z) == R.g1_affine(e), algo


def test_zkfc_and_tlookup():
    rng = random.Random(2)
    B, I, O = 3, 5, 7
    X, W = rand_small_fr(rng, B * I), rand_small_fr(rng, I * O)
    Y = R.matmul(X, W, B, I, O)
    ub, ui, uo = rand_fr(rng, 2), rand_fr(rng, 3), rand_fr(rng, 3)
    exp = R.zkfc_prove(X, W, Y, B, I, O, ub, ui, uo)
    rc, polys, claims = C.zkfc_prove(R.fr_pack(X), R.fr_pack(W), R.fr_pack(Y), B, I, O, R.fr_pack(ub), R.fr_pack(ui), R.fr_pack(uo))
    assert rc == 0
    p = R.fr_unpack(polys)
    assert [p[3 * i:3 * i + 3] for i in range(3)] == exp["proof"]
    assert R.fr_unpack(claims) == [exp["claim"], exp["final_claim"], exp["claim_x"], exp["claim_w"]]
    for D, N in ((64, 8), (16, 16), (8, 1)):
        low = -2
        table = R.range_table(low, N)
        vals = [R.int_to_fr(rng.randrange(low, low + N)) for _ in range(D)]
        m = R.tlookup_prep(R.range_indices(vals, low), N)
        k = R.ceil_log2(D)
        alpha, beta, u, v = rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rand_fr(rng, k), rand_fr(rng, k)
        exp_p = []
        exp_c = R.tlookup_prove(vals, table, m, alpha, beta, u, v, exp_p)
        rc, polys, final = C.tlookup_prove(R.fr_pack(vals), R.fr_pack(table), R.fr_pack(m), R.fr_pack([alpha]), R.fr_pack([beta]),
                                           R.fr_pack(u), R.fr_pack(v))
        assert rc == 0
        p = R.fr_unpack(polys)
        assert [p[4 * i:4 * i + 4] for i in range(k)] == [(q + [0, 0, 0, 0])[:4] for q in exp_p]
        assert R.fr_unpack(final)[0] == exp_c


def test_me_open():
    rng = random.Random(5)
    for n, k in [(1, 0), (5, 3), (8, 3)]:
        gens = seeded_generators(n, 40 + n)
        t, u = rand_fr(rng, n), rand_fr(rng, k)
        proof = []
        exp = R.me_open(t, gens, u, proof)
        got_proof, got = C.me_open(R.fr_pack(t), R.g1_pack(gens), R.fr_pack(u) if k else np.zeros((0, 8), dtype=np.uint32))
        assert R.fr_unpack(got)[0] == exp
        assert [R.g1_affine(p) for p in R.g1_unpack(got_proof)] == [R.g1_affine(p) for p in proof]
