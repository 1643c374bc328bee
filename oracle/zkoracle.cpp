// TEST INFRASTRUCTURE ONLY - CPU restatement of the reference prover path, used by
// tests/ as the checker at sizes where the Python oracle is too slow, and by
// bench.py as the timed CPU baseline.  The product library never links or calls it.
//
// Binary layouts are the reference's: Fr = 32-byte little-endian standard form,
// G1 = Jacobian (X, Y, Z) of 48-byte Montgomery-form Fq (bls12-381.cuh:116-120,
// 424-433).  Every function names the reference code it restates.
//
// Parity status: pinned through oracle/pyref.py (tests/test_oracle_cpp.py checks
// this file against it; tests/test_oracle_golden.py checks pyref against outputs
// of the reference's own CUDA build).
#include "zkoracle.h"

#include <omp.h>

#include <cstdlib>
#include <vector>

#include "bigfield.hpp"

using namespace zko;

namespace {

inline FrE ld_fr(const uint32_t* p) { FrE r; std::memcpy(r.l, p, 32); return r; }
inline void st_fr(uint32_t* p, const FrE& a) { std::memcpy(p, a.l, 32); }
inline G1 ld_g1(const uint32_t* p) { G1 r; std::memcpy(&r, p, 144); return r; }
inline void st_g1(uint32_t* p, const G1& a) { std::memcpy(p, &a, 144); }

inline FrE fr_from_i64(long long v) {
    if (v >= 0) return Fr::from_u64((uint64_t)v);
    return Fr::neg(Fr::from_u64(0ull - (uint64_t)v));
}
inline FrE fmul(const FrE& a, const FrE& b) { return Fr::mul_std(a, b); }

unsigned clog2(size_t n) { unsigned r = 0; if (!n) return 0; --n; while (n) { n >>= 1; ++r; } return r; }

// LSB-first multilinear fold of one axis, in place semantics of Fr_me_step (fr-tensor.cu:588-600)
std::vector<FrE> me_step(const std::vector<FrE>& t, const FrE& x) {
    std::vector<FrE> out((t.size() + 1) / 2);
    const FrE xm = Fr::to_mont(x);
    for (size_t i = 0; i < out.size(); ++i) {
        const FrE a0 = t[2 * i];
        const FrE a1 = (2 * i + 1 < t.size()) ? t[2 * i + 1] : Fr::zero();
        out[i] = Fr::add(a0, Fr::mmul(xm, Fr::sub(a1, a0)));
    }
    return out;
}
FrE mle_eval(std::vector<FrE> t, const FrE* u, unsigned k) {
    for (unsigned i = 0; i < k; ++i) t = me_step(t, u[i]);
    return t[0];
}
// FrTensor::partial_me(u, cur_dim, window) (fr-tensor.cu:518-560)
std::vector<FrE> partial_me(std::vector<FrE> t, const FrE* u, unsigned k, size_t cur, size_t window) {
    for (unsigned r = 0; r < k; ++r) {
        const size_t other = t.size() / (cur * window), od = (cur + 1) / 2;
        std::vector<FrE> out(other * od * window);
        const FrE xm = Fr::to_mont(u[r]);
        for (size_t o = 0; o < other; ++o)
            for (size_t j = 0; j < od; ++j)
                for (size_t w = 0; w < window; ++w) {
                    const FrE a0 = t[o * cur * window + (2 * j) * window + w];
                    const FrE a1 = (2 * j + 1 < cur) ? t[o * cur * window + (2 * j + 1) * window + w] : Fr::zero();
                    out[(o * od + j) * window + w] = Fr::add(a0, Fr::mmul(xm, Fr::sub(a1, a0)));
                }
        t.swap(out);
        cur = od;
    }
    return t;
}
FrE poly_eval(const FrE* c, int n, const FrE& x) {
    FrE acc = Fr::zero();
    for (int i = n - 1; i >= 0; --i) acc = Fr::add(fmul(acc, x), c[i]);
    return acc;
}
FrE eq_eval(const FrE& u, const FrE& v) {   // polynomial.cu:355-360
    FrE uv = fmul(u, v);
    return Fr::add(Fr::sub(Fr::dbl(uv), Fr::add(u, v)), Fr::from_u64(1));
}

// zkip (zkfc.cu:94-151); returns 0, or 1 when a round check fails
int zkip(FrE claim, std::vector<FrE> a, std::vector<FrE> b, const FrE* u, unsigned k, FrE* polys, FrE* final_claim) {
    for (unsigned r = 0; r < k; ++r) {
        const size_t n_in = a.size(), n_out = ((size_t)1 << clog2(n_in)) >> 1;
        const FrE v = u[k - 1 - r], vm = Fr::to_mont(v);
        FrE c0 = Fr::zero(), c1 = Fr::zero(), c2 = Fr::zero();
        std::vector<FrE> na(n_out), nb(n_out);
        for (size_t g = 0; g < n_out; ++g) {
            const FrE a0 = g < n_in ? a[g] : Fr::zero(), b0 = g < n_in ? b[g] : Fr::zero();
            const FrE a1 = g + n_out < n_in ? a[g + n_out] : Fr::zero(), b1 = g + n_out < n_in ? b[g + n_out] : Fr::zero();
            const FrE da = Fr::sub(a1, a0), db = Fr::sub(b1, b0);
            c0 = Fr::add(c0, fmul(a0, b0));
            c1 = Fr::add(c1, Fr::add(fmul(a0, db), fmul(b0, da)));
            c2 = Fr::add(c2, fmul(da, db));
            na[g] = Fr::add(a0, Fr::mmul(vm, da));
            nb[g] = Fr::add(b0, Fr::mmul(vm, db));
        }
        polys[3 * r] = c0; polys[3 * r + 1] = c1; polys[3 * r + 2] = c2;
        const FrE p1 = Fr::add(Fr::add(c0, c1), c2);
        if (!Fr::eq(claim, Fr::add(c0, p1))) return 1;
        claim = poly_eval(polys + 3 * r, 3, v);
        a.swap(na); b.swap(nb);
    }
    *final_claim = claim;
    return 0;
}

// ---- MSM ---------------------------------------------------------------------------
// commit_int_dev_func (commitment.cu:31-42): 31 x {conditional add; double}, then
// subtract 2^31 * a when the int is negative.
G1 commit_term_ref(G1 a, int x) {
    G1 out = g1_zero();
    for (unsigned i = 0; i < 31; ++i) {
        if ((x >> i) & 1) out = g1_add(out, a);
        a = g1_double(a);
    }
    if (x < 0) out = g1_add(out, g1_neg(a));
    return out;
}

// Signed 7-bit-window bucket method for one row (the algorithm the CUDA core uses).
G1 msm_row_pippenger(const std::vector<G1A>& bases, const int32_t* s, size_t n, int W) {
    const int c = 7, nb = 64;
    G1 acc = g1_zero();
    std::vector<G1> buckets(nb);
    for (int w = W - 1; w >= 0; --w) {
        for (int d = 0; d < c && w != W - 1; ++d) acc = g1_double(acc);
        for (int b = 0; b < nb; ++b) buckets[b] = g1_zero();
        for (size_t j = 0; j < n; ++j) {
            const int v = s[j];
            const uint64_t a = v < 0 ? 0ull - (uint64_t)(int64_t)v : (uint64_t)v;
            uint64_t K = 0;
            for (int q = 0; q < 9; ++q) K |= 64ull << (c * q);
            int d = (int)(((a + K) >> (c * w)) & 127u) - 64;
            if (v < 0) d = -d;
            if (!d) continue;
            buckets[(d < 0 ? -d : d) - 1] = g1_add_affine(buckets[(d < 0 ? -d : d) - 1], d < 0 ? g1a_neg(bases[j]) : bases[j]);
        }
        G1 run = g1_zero(), tot = g1_zero();
        for (int b = nb - 1; b >= 0; --b) { run = g1_add(run, buckets[b]); tot = g1_add(tot, run); }
        acc = g1_add(acc, tot);
    }
    return acc;
}

}  // namespace

extern "C" {

int zko_threads(void) { return omp_get_max_threads(); }

void zko_fr_mul(const uint32_t* a, const uint32_t* b, uint32_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) st_fr(out + 8 * i, fmul(ld_fr(a + 8 * i), ld_fr(b + 8 * i)));
}
void zko_fr_inv(const uint32_t* a, uint32_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) st_fr(out + 8 * i, Fr::inv_std(ld_fr(a + 8 * i)));
}
void zko_g1_add(const uint32_t* a, const uint32_t* b, uint32_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) st_g1(out + 36 * i, g1_add(ld_g1(a + 36 * i), ld_g1(b + 36 * i)));
}
void zko_g1_to_affine_jac(const uint32_t* a, uint32_t* out, size_t n) {
    // normalised Jacobian (x, y, 1) or all-zero for the identity
    for (size_t i = 0; i < n; ++i) {
        G1A p = g1_to_affine(ld_g1(a + 36 * i));
        G1 r = g1_zero();
        if (!p.inf) { r.x = p.x; r.y = p.y; r.z = Fq::to_mont(Fq::from_u64(1)); }
        st_g1(out + 36 * i, r);
    }
}
// G1Jacobian_mul (g1-tensor.cu:445-453)
void zko_g1_mul(const uint32_t* g, const uint32_t* k, uint32_t* out, size_t n) {
#pragma omp parallel for schedule(dynamic)
    for (long i = 0; i < (long)n; ++i) {
        G1 a = ld_g1(g + 36 * i), acc = g1_zero();
        FrE s = ld_fr(k + 8 * i);
        for (int bit = 0; bit < 256; ++bit) {
            if ((s.l[bit >> 6] >> (bit & 63)) & 1) acc = g1_add(acc, a);
            a = g1_double(a);
        }
        st_g1(out + 36 * i, acc);
    }
}

// Commitment::commit_int (commitment.cu:31-58), the reference's own algorithm:
// one double-and-add per (row, generator) pair, then the row sum.
void zko_commit_int_ref(const uint32_t* gens, size_t n, const int32_t* scalars, size_t m, uint32_t* out, int threads) {
    std::vector<G1> g(n);
    for (size_t j = 0; j < n; ++j) g[j] = ld_g1(gens + 36 * j);
#pragma omp parallel for schedule(dynamic) num_threads(threads > 0 ? threads : omp_get_max_threads())
    for (long r = 0; r < (long)m; ++r) {
        G1 acc = g1_zero();
        for (size_t j = 0; j < n; ++j) acc = g1_add(acc, commit_term_ref(g[j], scalars[(size_t)r * n + j]));
        st_g1(out + 36 * r, acc);
    }
}

// Same result through the signed-digit bucket method (the CUDA core's algorithm).
void zko_commit_int_pippenger(const uint32_t* gens, size_t n, const int32_t* scalars, size_t m, uint32_t* out, int threads) {
    std::vector<G1A> bases(n);
    for (size_t j = 0; j < n; ++j) bases[j] = g1_to_affine(ld_g1(gens + 36 * j));
    uint64_t mx = 0;
    for (size_t i = 0; i < m * n; ++i) {
        const int v = scalars[i];
        const uint64_t a = v < 0 ? 0ull - (uint64_t)(int64_t)v : (uint64_t)v;
        if (a > mx) mx = a;
    }
    int W = 9;
    { uint64_t p = 128; for (int w = 1; w < 9; ++w, p *= 128) if (mx * 127 < 63 * p + 64) { W = w; break; } }
#pragma omp parallel for schedule(dynamic) num_threads(threads > 0 ? threads : omp_get_max_threads())
    for (long r = 0; r < (long)m; ++r) st_g1(out + 36 * r, msm_row_pippenger(bases, scalars + (size_t)r * n, n, W));
}

// scalar product by the raw bits of k, as G1Jacobian_mul does (g1-tensor.cu:445-453)
static G1 g1_mul_raw(G1 a, const FrE& k) {
    G1 acc = g1_zero();
    for (int bit = 0; bit < 256; ++bit) {
        if ((k.l[bit >> 6] >> (bit & 63)) & 1) acc = g1_add(acc, a);
        a = g1_double(a);
    }
    return acc;
}

// Commitment::me_open with me_open_step's five products per pair (commitment.cu:79-125).
void zko_me_open(const uint32_t* t, const uint32_t* gens, size_t n, const uint32_t* u, unsigned k, uint32_t* proof, uint32_t* out) {
    std::vector<FrE> sc(n);
    std::vector<G1> g(n);
    for (size_t i = 0; i < n; ++i) { sc[i] = ld_fr(t + 8 * i); g[i] = ld_g1(gens + 36 * i); }
    for (unsigned r = 0; r < k; ++r) {
        const size_t cur = sc.size(), nn = (cur + 1) / 2;
        const FrE us = ld_fr(u + 8 * r), um = Fr::to_mont(us);
        std::vector<FrE> ns(nn);
        std::vector<G1> ng(nn), a(nn), a0(nn), a1(nn);
#pragma omp parallel for schedule(dynamic)
        for (long j = 0; j < (long)nn; ++j) {
            const size_t i0 = 2 * j, i1 = 2 * j + 1;
            if (i1 >= cur) {
                ns[j] = Fr::sub(sc[i0], Fr::mmul(um, sc[i0]));
                ng[j] = g1_mul_raw(g[i0], us);
                a[j] = g1_mul_raw(g[i0], sc[i0]);
                a0[j] = g1_zero();
                a1[j] = g1_zero();
                continue;
            }
            ns[j] = Fr::add(sc[i0], Fr::mmul(um, Fr::sub(sc[i1], sc[i0])));
            ng[j] = g1_add(g[i1], g1_mul_raw(g1_add(g[i0], g1_neg(g[i1])), us));
            a[j] = g1_add(g1_mul_raw(g[i0], sc[i0]), g1_mul_raw(g[i1], sc[i1]));
            a0[j] = g1_mul_raw(g[i1], sc[i0]);
            a1[j] = g1_mul_raw(g[i0], sc[i1]);
        }
        G1 s = g1_zero(), s0 = g1_zero(), s1 = g1_zero();
        for (size_t j = 0; j < nn; ++j) { s = g1_add(s, a[j]); s0 = g1_add(s0, a0[j]); s1 = g1_add(s1, a1[j]); }
        st_g1(proof + 36 * (3 * r), s);
        st_g1(proof + 36 * (3 * r + 1), s0);
        st_g1(proof + 36 * (3 * r + 2), s1);
        sc.swap(ns);
        g.swap(ng);
    }
    st_g1(proof + 36 * 3 * (size_t)k, g[0]);
    st_fr(out, sc[0]);
}

void zko_mle_eval(const uint32_t* a, size_t n, const uint32_t* u, unsigned k, uint32_t* out) {
    std::vector<FrE> t(n), uu(k);
    for (size_t i = 0; i < n; ++i) t[i] = ld_fr(a + 8 * i);
    for (unsigned i = 0; i < k; ++i) uu[i] = ld_fr(u + 8 * i);
    st_fr(out, mle_eval(t, uu.data(), k));
}

int zko_zkip(const uint32_t* claim, const uint32_t* a, const uint32_t* b, size_t n, const uint32_t* u, unsigned k,
             uint32_t* polys, uint32_t* final_claim) {
    std::vector<FrE> va(n), vb(n), uu(k), pp(3 * (size_t)k + 1);
    for (size_t i = 0; i < n; ++i) { va[i] = ld_fr(a + 8 * i); vb[i] = ld_fr(b + 8 * i); }
    for (unsigned i = 0; i < k; ++i) uu[i] = ld_fr(u + 8 * i);
    FrE fc;
    int rc = zkip(ld_fr(claim), va, vb, uu.data(), k, pp.data(), &fc);
    if (rc) return rc;
    for (size_t i = 0; i < 3 * (size_t)k; ++i) st_fr(polys + 8 * i, pp[i]);
    st_fr(final_claim, fc);
    return 0;
}

// body of zkFC::prove (zkfc.cu:61-87) with the reference's fold order.
// claims = {claim, final_claim, claim_X, claim_W}; returns 0, 1 (round check), 2 (final check)
int zko_zkfc_prove(const uint32_t* X, const uint32_t* Wt, const uint32_t* Y, size_t B, size_t I, size_t O,
                   const uint32_t* ub, const uint32_t* ui, const uint32_t* uo, uint32_t* polys, uint32_t* claims) {
    const unsigned kB = clog2(B), kI = clog2(I), kO = clog2(O);
    std::vector<FrE> x(B * I), w(I * O), y(B * O), vb(kB), vi(kI), vo(kO);
    for (size_t i = 0; i < x.size(); ++i) x[i] = ld_fr(X + 8 * i);
    for (size_t i = 0; i < w.size(); ++i) w[i] = ld_fr(Wt + 8 * i);
    for (size_t i = 0; i < y.size(); ++i) y[i] = ld_fr(Y + 8 * i);
    for (unsigned i = 0; i < kB; ++i) vb[i] = ld_fr(ub + 8 * i);
    for (unsigned i = 0; i < kI; ++i) vi[i] = ld_fr(ui + 8 * i);
    for (unsigned i = 0; i < kO; ++i) vo[i] = ld_fr(uo + 8 * i);
    const FrE claim = mle_eval(partial_me(y, vo.data(), kO, O, 1), vb.data(), kB);
    std::vector<FrE> xr = partial_me(x, vb.data(), kB, B, I);
    std::vector<FrE> wr = partial_me(w, vo.data(), kO, O, 1);
    std::vector<FrE> pp(3 * (size_t)kI + 1);
    FrE fc;
    if (zkip(claim, xr, wr, vi.data(), kI, pp.data(), &fc)) return 1;
    const FrE cx = mle_eval(partial_me(x, vi.data(), kI, I, 1), vb.data(), kB);
    const FrE cw = mle_eval(partial_me(w, vo.data(), kO, O, 1), vi.data(), kI);
    for (size_t i = 0; i < 3 * (size_t)kI; ++i) st_fr(polys + 8 * i, pp[i]);
    st_fr(claims, claim); st_fr(claims + 8, fc); st_fr(claims + 16, cx); st_fr(claims + 24, cw);
    return Fr::eq(fmul(cx, cw), fc) ? 0 : 2;
}

// tLookup::prove (tlookup.cu:184-370).  polys: 4 coefficients per round.
// Returns 0, or 1/2 when a phase-1/phase-2 round check fails.
int zko_tlookup_prove(const uint32_t* S_, const uint32_t* T_, const uint32_t* m_, size_t D, size_t N,
                      const uint32_t* alpha_, const uint32_t* beta_, const uint32_t* u_, const uint32_t* v_,
                      uint32_t* polys, uint32_t* final_claim, int threads) {
    const unsigned kD = clog2(D), kN = clog2(N), k1 = kD - kN;
    const int nt = threads > 0 ? threads : omp_get_max_threads();
    std::vector<FrE> S(D), A(D), T(N), Bv(N), m(N), u(kD), v(kD);
    const FrE beta = ld_fr(beta_);
    FrE alpha = ld_fr(alpha_);
    for (size_t i = 0; i < N; ++i) { T[i] = ld_fr(T_ + 8 * i); m[i] = ld_fr(m_ + 8 * i); Bv[i] = Fr::inv_std(Fr::add(T[i], beta)); }
#pragma omp parallel for num_threads(nt)
    for (long i = 0; i < (long)D; ++i) { S[i] = ld_fr(S_ + 8 * i); A[i] = Fr::inv_std(Fr::add(S[i], beta)); }
    for (unsigned i = 0; i < kD; ++i) { u[i] = ld_fr(u_ + 8 * i); v[i] = ld_fr(v_ + 8 * i); }
    FrE bm = Fr::zero();
    for (size_t i = 0; i < N; ++i) bm = Fr::add(bm, fmul(Bv[i], m[i]));
    FrE alpha_sq = fmul(alpha, alpha);
    FrE C = Fr::sub(alpha_sq, bm);
    FrE claim = Fr::add(alpha, alpha_sq);
    const FrE two_inv = Fr::inv_std(Fr::from_u64(2));
    const FrE inv_ratio = fmul(Fr::from_u64(N), Fr::inv_std(Fr::from_u64(D)));
    unsigned nu = kD;
    size_t M = D;
    auto eq_table = [&](unsigned k) {   // eq(u[0..k), i), LSB first, standard form
        std::vector<FrE> e(1, Fr::from_u64(1));
        for (unsigned j = 0; j < k; ++j) {
            std::vector<FrE> ne(e.size() * 2);
            const FrE one_minus = Fr::sub(Fr::from_u64(1), u[j]);
            for (size_t i = 0; i < e.size(); ++i) { ne[i] = fmul(e[i], one_minus); ne[i + e.size()] = fmul(e[i], u[j]); }
            e.swap(ne);
        }
        return e;
    };
    for (unsigned r = 0; r < kD; ++r) {
        const size_t half = M / 2;
        const std::vector<FrE> e = eq_table(nu - 1);
        const FrE ub = u[nu - 1];
        const FrE e0 = Fr::sub(Fr::from_u64(1), ub), e1 = Fr::sub(Fr::dbl(ub), Fr::from_u64(1));
        const bool ph1 = r < k1;
        const FrE vb = ph1 ? v[k1 - 1 - r] : v[kD - 1 - (r - k1)];
        const FrE vm = Fr::to_mont(vb);
        FrE q[11];
        for (int i = 0; i < 11; ++i) q[i] = Fr::zero();
        std::vector<FrE> nA(half), nS(half), nB, nT, nm;
        if (!ph1) { nB.resize(half); nT.resize(half); nm.resize(half); }
#pragma omp parallel num_threads(nt)
        {
            FrE lq[11];
            for (int i = 0; i < 11; ++i) lq[i] = Fr::zero();
#pragma omp for nowait
            for (long ii = 0; ii < (long)half; ++ii) {
                const size_t i = (size_t)ii;
                const FrE ee = e[i];
                auto term = [&](const FrE& x0, const FrE& x1, const FrE& y0, const FrE& y1, FrE* o) {
                    const FrE c01 = Fr::sub(x1, x0), c10 = Fr::add(y0, beta), c11 = Fr::sub(y1, y0);
                    o[0] = Fr::add(o[0], fmul(ee, fmul(x0, c10)));
                    o[1] = Fr::add(o[1], fmul(ee, Fr::add(fmul(c01, c10), fmul(x0, c11))));
                    o[2] = Fr::add(o[2], fmul(ee, fmul(c01, c11)));
                };
                term(A[i], A[i + half], S[i], S[i + half], lq);
                lq[6] = Fr::add(lq[6], A[i]);
                lq[7] = Fr::add(lq[7], Fr::sub(A[i + half], A[i]));
                nA[i] = Fr::add(A[i], Fr::mmul(vm, Fr::sub(A[i + half], A[i])));
                nS[i] = Fr::add(S[i], Fr::mmul(vm, Fr::sub(S[i + half], S[i])));
                if (!ph1) {
                    term(Bv[i], Bv[i + half], T[i], T[i + half], lq + 3);
                    const FrE m0 = m[i], m1 = Fr::sub(m[i + half], m[i]), b0 = Bv[i], b1 = Fr::sub(Bv[i + half], Bv[i]);
                    lq[8] = Fr::add(lq[8], fmul(m0, b0));
                    lq[9] = Fr::add(lq[9], Fr::add(fmul(m1, b0), fmul(m0, b1)));
                    lq[10] = Fr::add(lq[10], fmul(m1, b1));
                    nB[i] = Fr::add(b0, Fr::mmul(vm, b1));
                    nT[i] = Fr::add(T[i], Fr::mmul(vm, Fr::sub(T[i + half], T[i])));
                    nm[i] = Fr::add(m0, Fr::mmul(vm, m1));
                }
            }
#pragma omp critical
            for (int i = 0; i < 11; ++i) q[i] = Fr::add(q[i], lq[i]);
        }
        FrE p0[3], p[4];
        if (ph1) for (int i = 0; i < 3; ++i) p0[i] = fmul(alpha, q[i]);
        else {
            const FrE cB = fmul(inv_ratio, alpha_sq);
            for (int i = 0; i < 3; ++i) p0[i] = Fr::add(fmul(alpha, q[i]), fmul(cB, q[3 + i]));
        }
        p[0] = fmul(p0[0], e0);
        p[1] = Fr::add(fmul(p0[1], e0), fmul(p0[0], e1));
        p[2] = Fr::add(fmul(p0[2], e0), fmul(p0[1], e1));
        p[3] = fmul(p0[2], e1);
        if (ph1) {
            p[0] = Fr::add(Fr::add(p[0], q[6]), fmul(C, two_inv));
            p[1] = Fr::add(p[1], q[7]);
        } else {
            p[0] = Fr::sub(Fr::add(p[0], q[6]), fmul(q[8], inv_ratio));
            p[1] = Fr::sub(Fr::add(p[1], q[7]), fmul(q[9], inv_ratio));
            p[2] = Fr::sub(p[2], fmul(q[10], inv_ratio));
        }
        for (int i = 0; i < 4; ++i) st_fr(polys + 8 * (4 * (size_t)r + i), p[i]);
        const FrE at1 = Fr::add(Fr::add(p[0], p[1]), Fr::add(p[2], p[3]));
        if (!Fr::eq(claim, Fr::add(p[0], at1))) return ph1 ? 1 : 2;
        claim = poly_eval(p, 4, vb);
        const FrE ev = eq_eval(ub, vb);
        alpha = fmul(alpha, ev);
        if (ph1) C = fmul(C, two_inv); else alpha_sq = fmul(alpha_sq, ev);
        A.swap(nA); S.swap(nS);
        if (!ph1) { Bv.swap(nB); T.swap(nT); m.swap(nm); }
        M = half;
        --nu;
    }
    st_fr(final_claim, claim);
    return 0;
}

}  // extern "C"
