// Host side of the multi-GPU sumchecks: what every rank does with the gathered
// per-rank results of zkb_zkip_partial / zkb_tlookup_partial.  The vectors are dealt
// out round-robin (rank p holds the indices i = p mod P), every rank has run all
// its local rounds, and one all-gather has brought the blocks together.  Here the
// coefficient sums are added, the last log2(P) rounds run on the P surviving
// entries, the round polynomials are assembled and the reference's verifier
// checks are replayed (zkfc.cu:140-151, tlookup.cu:281-322).  Plain CPU arithmetic:
// a few thousand field products per proof.
#include "common.cuh"
#include "hostfr.hpp"

#include <vector>

using namespace zkb;
using hfr::H;

namespace {

inline unsigned log2u(size_t n) {
    unsigned r = 0;
    while (((size_t)1 << r) < n) ++r;
    return r;
}

// eq(u[0..nbits); index): challenge j pairs with bit j of the index
H eq_weight(const zkb_fr_t* u, unsigned nbits, size_t index) {
    H w = hfr::from_u64(1);
    const H one = hfr::from_u64(1);
    for (unsigned j = 0; j < nbits; ++j) {
        const H uj = hfr::load(u[j]);
        w = hfr::mul(w, ((index >> j) & 1) ? uj : hfr::sub(one, uj));
    }
    return w;
}

}  // namespace

extern "C" {

int zkb_zkip_combine(const zkb_fr_t* h_parts, unsigned world, unsigned k, const zkb_fr_t* h_u, const zkb_fr_t* h_claim,
                     zkb_fr_t* h_polys, zkb_fr_t* h_final) {
    if (!world || (world & (world - 1))) return fail(ZKB_ERR_ARG, "zkip: the number of ranks must be a power of two");
    const unsigned kP = log2u(world);
    if (k < kP) return fail(ZKB_ERR_DIM, "zkip: more ranks than entries");
    const unsigned local = k - kP;                       // rounds every rank ran on its own
    const size_t block = 3 * (size_t)local + 2;          // sums, then the rank's surviving pair (a, b)
    std::vector<H> polys(3 * (size_t)k, hfr::zero());
    for (unsigned p = 0; p < world; ++p)
        for (size_t i = 0; i < 3 * (size_t)local; ++i) polys[i] = hfr::add(polys[i], hfr::load(h_parts[p * block + i]));
    std::vector<H> a(world), b(world);
    for (unsigned p = 0; p < world; ++p) {
        a[p] = hfr::load(h_parts[p * block + 3 * local]);
        b[p] = hfr::load(h_parts[p * block + 3 * local + 1]);
    }
    for (unsigned r = local; r < k; ++r) {
        const H v = hfr::load(h_u[k - 1 - r]);
        const size_t half = a.size() / 2;
        H c0 = hfr::zero(), c1 = hfr::zero(), c2 = hfr::zero();
        std::vector<H> na(half), nb(half);
        for (size_t g = 0; g < half; ++g) {
            const H da = hfr::sub(a[g + half], a[g]), db = hfr::sub(b[g + half], b[g]);
            c0 = hfr::add(c0, hfr::mul(a[g], b[g]));
            c1 = hfr::add(c1, hfr::add(hfr::mul(a[g], db), hfr::mul(b[g], da)));
            c2 = hfr::add(c2, hfr::mul(da, db));
            na[g] = hfr::add(a[g], hfr::mul(v, da));
            nb[g] = hfr::add(b[g], hfr::mul(v, db));
        }
        polys[3 * r] = c0; polys[3 * r + 1] = c1; polys[3 * r + 2] = c2;
        a.swap(na);
        b.swap(nb);
    }
    H claim = hfr::load(*h_claim);
    for (unsigned r = 0; r < k; ++r) {
        const H* c = &polys[3 * r];
        for (int i = 0; i < 3; ++i) h_polys[3 * r + i] = hfr::store(c[i]);
        const H p1 = hfr::add(hfr::add(c[0], c[1]), c[2]);
        if (!hfr::eq(claim, hfr::add(c[0], p1))) return fail(ZKB_ERR_VERIFY, "claim != p(0) + p(1)");
        claim = hfr::poly_eval(c, 3, hfr::load(h_u[k - 1 - r]));
    }
    *h_final = hfr::store(claim);
    return ZKB_OK;
}

// Per-rank block of zkb_tlookup_combine: the 1 + 11 * local sums of zkb_tlookup_partial, then the
// rank's surviving entries A, S, B, T, m (one each).
int zkb_tlookup_combine(const zkb_fr_t* h_parts, unsigned world, size_t D, size_t N, const zkb_fr_t* h_alpha,
                        const zkb_fr_t* h_beta, const zkb_fr_t* h_u, const zkb_fr_t* h_v, zkb_fr_t* h_polys, zkb_fr_t* h_final) {
    if (!world || (world & (world - 1))) return fail(ZKB_ERR_ARG, "tLookup: the number of ranks must be a power of two");
    if (!D || !N || (D & (D - 1)) || (N & (N - 1)) || D % N)
        return fail(ZKB_ERR_DIM, "D or N is not power of 2, or D is not divisible by N");
    const unsigned kP = log2u(world), kD = log2u(D), kN = log2u(N), k1 = kD - kN;
    if (kN < kP) return fail(ZKB_ERR_DIM, "tLookup: more ranks than table entries");
    const unsigned local = kD - kP;
    const size_t block = 1 + 11 * (size_t)local + 5;
    // sums[0] = sum B*m; then 11 per round.  The eq-weighted slots of a rank carry the
    // weight of its own index bits, eq(u[0..kP); rank), as one common factor.
    std::vector<H> sums(1 + 11 * (size_t)kD, hfr::zero());
    for (unsigned p = 0; p < world; ++p) {
        const zkb_fr_t* part = h_parts + p * block;
        const H w = eq_weight(h_u, kP, p);
        sums[0] = hfr::add(sums[0], hfr::load(part[0]));
        for (unsigned r = 0; r < local; ++r) {
            const unsigned weighted = r < k1 ? 3 : 6;
            for (unsigned c = 0; c < 11; ++c) {
                const size_t i = 1 + 11 * (size_t)r + c;
                const H x = hfr::load(part[i]);
                sums[i] = hfr::add(sums[i], c < weighted ? hfr::mul(w, x) : x);
            }
        }
    }
    // the last kP rounds (all of phase 2) on the P surviving entries: entry of rank p is index p
    const H beta = hfr::load(*h_beta);
    std::vector<H> arr[5];
    for (int a = 0; a < 5; ++a) {
        arr[a].resize(world);
        for (unsigned p = 0; p < world; ++p) arr[a][p] = hfr::load(h_parts[p * block + 1 + 11 * (size_t)local + a]);
    }
    for (unsigned r = local; r < kD; ++r) {
        const size_t half = arr[0].size() / 2;
        const unsigned nbits = log2u(half);
        const H vv = hfr::load(h_v[kD - 1 - (r - k1)]);
        H q[11];
        for (auto& x : q) x = hfr::zero();
        std::vector<H> nxt[5];
        for (auto& x : nxt) x.resize(half);
        for (size_t g = 0; g < half; ++g) {
            const H e = eq_weight(h_u, nbits, g);
            const H a0 = arr[0][g], a1 = arr[0][g + half], s0 = arr[1][g], s1 = arr[1][g + half];
            const H c01 = hfr::sub(a1, a0), c10 = hfr::add(s0, beta), c11 = hfr::sub(s1, s0);
            const H ea0 = hfr::mul(e, a0), ec01 = hfr::mul(e, c01);
            q[0] = hfr::add(q[0], hfr::mul(ea0, c10));
            q[1] = hfr::add(q[1], hfr::add(hfr::mul(ea0, c11), hfr::mul(ec01, c10)));
            q[2] = hfr::add(q[2], hfr::mul(ec01, c11));
            q[6] = hfr::add(q[6], a0);
            q[7] = hfr::add(q[7], c01);
            nxt[0][g] = hfr::add(a0, hfr::mul(vv, c01));
            nxt[1][g] = hfr::add(s0, hfr::mul(vv, c11));
            const H b0 = arr[2][g], b1 = arr[2][g + half], t0 = arr[3][g], t1 = arr[3][g + half];
            const H m0 = arr[4][g], m1f = arr[4][g + half];
            const H d01 = hfr::sub(b1, b0), d10 = hfr::add(t0, beta), d11 = hfr::sub(t1, t0);
            const H eb0 = hfr::mul(e, b0), ed01 = hfr::mul(e, d01);
            q[3] = hfr::add(q[3], hfr::mul(eb0, d10));
            q[4] = hfr::add(q[4], hfr::add(hfr::mul(eb0, d11), hfr::mul(ed01, d10)));
            q[5] = hfr::add(q[5], hfr::mul(ed01, d11));
            const H m1 = hfr::sub(m1f, m0);
            q[8] = hfr::add(q[8], hfr::mul(m0, b0));
            q[9] = hfr::add(q[9], hfr::add(hfr::mul(m0, d01), hfr::mul(m1, b0)));
            q[10] = hfr::add(q[10], hfr::mul(m1, d01));
            nxt[2][g] = hfr::add(b0, hfr::mul(vv, d01));
            nxt[3][g] = hfr::add(t0, hfr::mul(vv, d11));
            nxt[4][g] = hfr::add(m0, hfr::mul(vv, m1));
        }
        for (unsigned c = 0; c < 11; ++c) sums[1 + 11 * (size_t)r + c] = q[c];
        for (int a = 0; a < 5; ++a) arr[a].swap(nxt[a]);
    }
    std::vector<zkb_fr_t> flat(sums.size());
    for (size_t i = 0; i < sums.size(); ++i) flat[i] = hfr::store(sums[i]);
    return tlookup_assemble(flat.data(), D, N, h_alpha, h_u, h_v, h_polys, h_final);
}

// Per-rank block: (kN - log2 world) * (K + 1) coefficient sums of the rank's own rounds, then its K surviving entries.
int zkb_multi_hadamard_combine(const zkb_fr_t* h_parts, unsigned world, unsigned K, unsigned kN, const zkb_fr_t* h_u,
                               const zkb_fr_t* h_v, const zkb_fr_t* h_claim, zkb_fr_t* h_polys, zkb_fr_t* h_final) {
    if (!world || (world & (world - 1))) return fail(ZKB_ERR_ARG, "multi_hadamard: the number of ranks must be a power of two");
    if (K < 1 || K > 6) return fail(ZKB_ERR_LIMIT, "multi_hadamard: between 1 and 6 tensors");
    const unsigned kP = log2u(world);
    if (kN < kP) return fail(ZKB_ERR_DIM, "multi_hadamard: more ranks than entries");
    const unsigned local = kN - kP, W = K + 1;
    const size_t block = (size_t)local * W + K;
    std::vector<H> polys((size_t)kN * W, hfr::zero());
    // a rank's sums carry eq over the variables above its index bits; the factor of the index bits is its weight
    for (unsigned p = 0; p < world; ++p) {
        const H w = eq_weight(h_u, kP, p);
        for (size_t i = 0; i < (size_t)local * W; ++i)
            polys[i] = hfr::add(polys[i], hfr::mul(w, hfr::load(h_parts[p * block + i])));
    }
    // the last log2(world) rounds on the `world` surviving entries of every tensor (entry p = rank p)
    std::vector<std::vector<H>> x(K, std::vector<H>(world));
    for (unsigned p = 0; p < world; ++p)
        for (unsigned j = 0; j < K; ++j) x[j][p] = hfr::load(h_parts[p * block + (size_t)local * W + j]);
    size_t M = world;
    for (unsigned r = local; r < kN; ++r) {
        const size_t half = M / 2;
        const unsigned below = kN - 1 - r;               // variables still unbound below this one
        const H v = hfr::load(h_v[kN - 1 - r]);
        std::vector<H> c(W, hfr::zero());
        for (size_t g = 0; g < half; ++g) {
            std::vector<H> prod(W, hfr::zero());         // prod_j (x_j[g] + t (x_j[g + half] - x_j[g]))
            prod[0] = hfr::from_u64(1);
            for (unsigned j = 0; j < K; ++j) {
                const H a0 = x[j][g], d = hfr::sub(x[j][g + half], x[j][g]);
                for (unsigned i = j + 1; i >= 1; --i) prod[i] = hfr::add(hfr::mul(prod[i], a0), hfr::mul(prod[i - 1], d));
                prod[0] = hfr::mul(prod[0], a0);
                x[j][g] = hfr::add(a0, hfr::mul(v, d));
            }
            const H e = eq_weight(h_u, below, g);
            for (unsigned i = 0; i < W; ++i) c[i] = hfr::add(c[i], hfr::mul(e, prod[i]));
        }
        for (unsigned i = 0; i < W; ++i) polys[(size_t)r * W + i] = c[i];
        M = half;
    }
    for (size_t i = 0; i < polys.size(); ++i) h_polys[i] = hfr::store(polys[i]);
    return hadamard_replay(h_claim, h_polys, K, kN, h_u, h_v, h_final);
}

}  // extern "C"

namespace zkb {

int hadamard_replay(const zkb_fr_t* h_claim, const zkb_fr_t* h_polys, unsigned K, unsigned kN, const zkb_fr_t* h_u,
                    const zkb_fr_t* h_v, zkb_fr_t* h_final) {
    H claim = hfr::load(*h_claim);
    std::vector<H> c(K + 1);
    for (unsigned r = 0; r < kN; ++r) {
        for (unsigned i = 0; i <= K; ++i) c[i] = hfr::load(h_polys[(size_t)r * (K + 1) + i]);
        const H ub = hfr::load(h_u[kN - 1 - r]);
        const H e0 = hfr::sub(hfr::from_u64(1), ub);
        const H e1 = hfr::sub(hfr::add(ub, ub), hfr::from_u64(1));
        // (c * eq)(0) + (c * eq)(1) = c(0) e0 + c(1) (e0 + e1)
        H c_at1 = hfr::zero();
        for (unsigned i = 0; i <= K; ++i) c_at1 = hfr::add(c_at1, c[i]);
        const H lhs = hfr::add(hfr::mul(c[0], e0), hfr::mul(c_at1, hfr::add(e0, e1)));
        if (!hfr::eq(claim, lhs)) return fail(ZKB_ERR_VERIFY, "multi_hadamard_sumchecks: claim != p(0) + p(1)");
        claim = hfr::poly_eval(c.data(), (int)K + 1, hfr::load(h_v[kN - 1 - r]));
    }
    *h_final = hfr::store(claim);
    return ZKB_OK;
}

// Round polynomials of the lookup sumcheck from the per-round sums, with the
// reference's checks (tlookup.cu:281-322): sums[0] = sum B*m, then 11 values per round
// as zkb_tlookup_partial documents them.  Shared by the single-GPU prover and the
// multi-GPU combine.
int tlookup_assemble(const zkb_fr_t* sums, size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_u,
                     const zkb_fr_t* h_v, zkb_fr_t* h_polys, zkb_fr_t* h_final) {
    const unsigned kD = log2u(D), kN = log2u(N), k1 = kD - kN;
    const H alpha0 = hfr::load(*h_alpha);
    const H two_inv = hfr::inv(hfr::from_u64(2));
    H alpha = alpha0;
    H alpha_sq = hfr::mul(alpha0, alpha0);
    H C = hfr::sub(alpha_sq, hfr::load(sums[0]));
    H claim = hfr::add(alpha0, alpha_sq);
    const H inv_ratio = hfr::mul(hfr::from_u64(N), hfr::inv(hfr::from_u64(D)));
    unsigned nu = kD;   // challenges of u still unbound
    for (unsigned r = 0; r < kD; ++r) {
        const zkb_fr_t* q = &sums[1 + 11 * (size_t)r];
        const H ub = hfr::load(h_u[nu - 1]);
        const H e0 = hfr::sub(hfr::from_u64(1), ub);                 // eq(u)(t) = e0 + e1 t
        const H e1 = hfr::sub(hfr::add(ub, ub), hfr::from_u64(1));
        H p0[3], p[4];
        H vb;
        if (r < k1) {
            for (int i = 0; i < 3; ++i) p0[i] = hfr::mul(alpha, hfr::load(q[i]));
            vb = hfr::load(h_v[k1 - 1 - r]);
        } else {
            const H coefB = hfr::mul(inv_ratio, alpha_sq);
            for (int i = 0; i < 3; ++i)
                p0[i] = hfr::add(hfr::mul(alpha, hfr::load(q[i])), hfr::mul(coefB, hfr::load(q[3 + i])));
            vb = hfr::load(h_v[kD - 1 - (r - k1)]);
        }
        // p0 * eq
        p[0] = hfr::mul(p0[0], e0);
        p[1] = hfr::add(hfr::mul(p0[1], e0), hfr::mul(p0[0], e1));
        p[2] = hfr::add(hfr::mul(p0[2], e0), hfr::mul(p0[1], e1));
        p[3] = hfr::mul(p0[2], e1);
        if (r < k1) {
            p[0] = hfr::add(hfr::add(p[0], hfr::load(q[3])), hfr::mul(C, two_inv));
            p[1] = hfr::add(p[1], hfr::load(q[4]));
        } else {
            p[0] = hfr::sub(hfr::add(p[0], hfr::load(q[6])), hfr::mul(hfr::load(q[8]), inv_ratio));
            p[1] = hfr::sub(hfr::add(p[1], hfr::load(q[7])), hfr::mul(hfr::load(q[9]), inv_ratio));
            p[2] = hfr::sub(p[2], hfr::mul(hfr::load(q[10]), inv_ratio));
        }
        for (int i = 0; i < 4; ++i) h_polys[4 * (size_t)r + i] = hfr::store(p[i]);
        const H at1 = hfr::add(hfr::add(p[0], p[1]), hfr::add(p[2], p[3]));
        if (!hfr::eq(claim, hfr::add(p[0], at1)))
            return fail(ZKB_ERR_VERIFY, r < k1 ? "tLookup_phase1: claim != p(0) + p(1)" : "tLookup_phase2: claim != p(0) + p(1)");
        claim = hfr::poly_eval(p, 4, vb);
        const H e = hfr::eq_eval(ub, vb);
        alpha = hfr::mul(alpha, e);
        if (r < k1) C = hfr::mul(C, two_inv);
        else alpha_sq = hfr::mul(alpha_sq, e);
        --nu;
    }
    *h_final = hfr::store(claim);
    return ZKB_OK;
}

}  // namespace zkb
