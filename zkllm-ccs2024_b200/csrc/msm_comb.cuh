// Row commitments with many rows over one generator set: combination tables.
//
// Commitment::commit_int (commitment.cu:31-58) commits every row of an m x n
// matrix of small signed integers to the same n generators.  When m is large
// the generators can be prepared once per call and shared by all rows:
//
//   * every scalar is written in signed 3-bit digits d in [-4, 3]
//     (s + K with K = 4 in every 3-bit field makes each digit an independent
//     bit-field read, negative scalars included);
//   * the generators are taken four at a time; for each such group a table
//     holds all 8^4 = 4096 sums  d0 g0 + d1 g1 + d2 g2 + d3 g3  as affine
//     points, built from 64-entry tables of the two pairs with one affine
//     addition per entry (Montgomery's trick: one inversion per 64 entries);
//   * a row then needs ONE mixed addition per (window, group of four
//     generators): W/4 additions per (scalar, generator) pair instead of one
//     per 7-bit window, and no sorting, buckets or bucket reduction.  The 3-bit
//     windows are combined by doublings at the end.
//
// The tables cost ceil(n/4) * 4096 affine additions and 96 bytes per entry, so the
// caller chooses this path only when the rows outweigh that (see commit_i32_device).
#pragma once
#include "g1.cuh"

namespace zkb {

static constexpr int kCombBits = 3;
static constexpr unsigned kCombEntries = 4096;   // 8^4 digit combinations of four generators
static constexpr unsigned kCombZeroIdx = 0x924;  // field value 4 (digit 0) in all four positions
static constexpr int kCombMaxWindows = 11;       // int32: |s| <= (3 * 8^11 - 3) / 7

__host__ __device__ constexpr unsigned long long comb_bias(int W) {
    unsigned long long k = 0;
    for (int w = 0; w < W; ++w) k |= 4ull << (kCombBits * w);
    return k;
}
// Smallest W with s + K in [0, 8^W) for every |s| <= max_abs:  max_abs <= (3 * 8^W - 3) / 7.
static int comb_windows_for_max(unsigned long long max_abs) {
    unsigned long long p = 8;
    for (int W = 1; W < kCombMaxWindows; ++W, p *= 8)
        if (max_abs * 7 + 3 <= 3 * p) return W;
    return kCombMaxWindows;
}

ZKB_DEV G1Aff g1_aff_identity() {
    G1Aff r;
    r.x = fe_zero<FqParams>(); r.y = fe_zero<FqParams>();
    return r;
}

// ---- affine + affine with a shared inversion ---------------------------------------
// What a + b needs: the denominator of the chord (or tangent) slope, or no division at all.
enum { kAddChord = 0, kAddTangent = 1, kAddToIdentity = 2, kAddTakeB = 3, kAddTakeA = 4 };
ZKB_DEV int aff_add_kind(const G1Aff& a, const G1Aff& b, Fq& den) {
    if (g1_aff_is_identity(a)) return kAddTakeB;
    if (g1_aff_is_identity(b)) return kAddTakeA;
    den = fq_sub(b.x, a.x);
    if (!fe_is_zero(den)) return kAddChord;
    if (fe_eq(a.y, b.y) && !fe_is_zero(a.y)) {
        den = fq_dbl(a.y);
        return kAddTangent;
    }
    return kAddToIdentity;
}

// out(i) = A(i) + B(i) for i < K in one thread: denominators multiplied up, one
// inversion, then walked back (5M + 1S per addition).  `prefix` is thread-private.
template <int K, class FA, class FB, class FO>
ZKB_DEV void batch_affine_add(FA get_a, FB get_b, FO put, Fq* prefix) {
    Fq run = fe_mont_one<FqParams>();
#pragma unroll 1
    for (int i = 0; i < K; ++i) {
        const G1Aff a = get_a(i), b = get_b(i);
        Fq den;
        const int kind = aff_add_kind(a, b, den);
        prefix[i] = run;
        if (kind <= kAddTangent) run = fq_mul(run, den);
    }
    Fq inv = mont_inv<FqParams>(run);
#pragma unroll 1
    for (int i = K - 1; i >= 0; --i) {
        const G1Aff a = get_a(i), b = get_b(i);
        Fq den;
        const int kind = aff_add_kind(a, b, den);
        G1Aff r;
        if (kind <= kAddTangent) {
            const Fq di = fq_mul(inv, prefix[i]);
            inv = fq_mul(inv, den);
            Fq num;
            if (kind == kAddChord) {
                num = fq_sub(b.y, a.y);
            } else {
                const Fq xx = fq_sqr(a.x);
                num = fq_add(fq_dbl(xx), xx);
            }
            const Fq lam = fq_mul(num, di);
            r.x = fq_sub(fq_sub(fq_sqr(lam), a.x), b.x);
            r.y = fq_sub(fq_mul(lam, fq_sub(a.x, r.x)), a.y);
        } else if (kind == kAddTakeB) {
            r = b;
        } else if (kind == kAddTakeA) {
            r = a;
        } else {
            r = g1_aff_identity();
        }
        put(i, r);
    }
}

// singles[j*8 + f] = (f - 4) g_j for f = 0..7, affine.  Columns at or beyond n (padding of the
// last group of four) hold the identity.
__global__ void __launch_bounds__(128) comb_singles_kernel(const G1Aff* __restrict__ bases, size_t n, size_t n_pad,
                                                            G1Aff* __restrict__ singles) {
    const size_t j = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (j >= n_pad) return;
    G1Aff* out = singles + j * 8;
    G1Aff g = g1_aff_identity();
    if (j < n) g = g1_aff_load(bases + j);
    G1Aff mult[4];                       // 1g .. 4g
    mult[0] = g;
    if (g1_aff_is_identity(g)) {
        mult[1] = g; mult[2] = g; mult[3] = g;
    } else {
        G1Jac jac[3];
        G1Jac one;
        one.x = g.x; one.y = g.y; one.z = fe_mont_one<FqParams>();
        jac[0] = g1_double(one);
        jac[1] = g1_add_mixed(jac[0], g);
        jac[2] = g1_double(jac[0]);
        Fq pre[3], run = fe_mont_one<FqParams>();
#pragma unroll 1
        for (int i = 0; i < 3; ++i) {
            pre[i] = run;
            if (!g1_is_identity(jac[i])) run = fq_mul(run, jac[i].z);
        }
        Fq inv = mont_inv<FqParams>(run);
#pragma unroll 1
        for (int i = 2; i >= 0; --i) {
            if (g1_is_identity(jac[i])) {
                mult[i + 1] = g1_aff_identity();
                continue;
            }
            const Fq zi = fq_mul(inv, pre[i]);
            inv = fq_mul(inv, jac[i].z);
            const Fq zi2 = fq_sqr(zi);
            mult[i + 1].x = fq_mul(jac[i].x, zi2);
            mult[i + 1].y = fq_mul(jac[i].y, fq_mul(zi2, zi));
        }
    }
    g1_aff_store(out + 4, g1_aff_identity());
#pragma unroll 1
    for (int k = 1; k <= 4; ++k) {
        if (k <= 3) g1_aff_store(out + 4 + k, mult[k - 1]);
        g1_aff_store(out + 4 - k, g1_aff_neg(mult[k - 1]));
    }
}

// pairs[p*64 + fa + 8 fb] = singles[2p][fa] + singles[2p+1][fb].  Thread per (p, fb), eight additions.
__global__ void __launch_bounds__(128) comb_pairs_kernel(const G1Aff* __restrict__ singles, size_t n_pairs,
                                                          G1Aff* __restrict__ pairs) {
    const size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (t >= n_pairs * 8) return;
    const size_t p = t >> 3;
    const unsigned fb = (unsigned)(t & 7);
    const G1Aff* sa = singles + (2 * p) * 8;
    const G1Aff b = g1_aff_load(singles + (2 * p + 1) * 8 + fb);
    G1Aff* out = pairs + p * 64 + fb * 8;
    Fq prefix[8];
    batch_affine_add<8>([&](int i) { return g1_aff_load(sa + i); }, [&](int) { return b; },
                        [&](int i, const G1Aff& r) { g1_aff_store(out + i, r); }, prefix);
}

// table[q*4096 + lo + 64 hi] = pairs[2q][lo] + pairs[2q+1][hi].  Thread per (q, hi), 64 additions.
__global__ void __launch_bounds__(128) comb_quads_kernel(const G1Aff* __restrict__ pairs, size_t n_quads,
                                                          G1Aff* __restrict__ table) {
    const size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (t >= n_quads * 64) return;
    const size_t q = t >> 6;
    const unsigned hi = (unsigned)(t & 63);
    const G1Aff* pa = pairs + (2 * q) * 64;
    const G1Aff b = g1_aff_load(pairs + (2 * q + 1) * 64 + hi);
    G1Aff* out = table + q * kCombEntries + hi * 64;
    Fq prefix[64];
    batch_affine_add<64>([&](int i) { return g1_aff_load(pa + i); }, [&](int) { return b; },
                         [&](int i, const G1Aff& r) { g1_aff_store(out + i, r); }, prefix);
}

// ---- the rows ---------------------------------------------------------------------------
struct CombShape {
    size_t m, n;          // rows, generators
    size_t n_quads;       // ceil(n / 4)
    unsigned nseg;        // chains per (row, window)
    unsigned qps;         // groups of four per chain
    int W;                // 3-bit windows
};

// Table index of group q in window w for one row: the four 3-bit fields side by side.
ZKB_DEV unsigned comb_index(const int32_t* __restrict__ row, size_t n, size_t q, int w, unsigned long long bias, bool vec) {
    int s0, s1 = 0, s2 = 0, s3 = 0;
    const size_t c = 4 * q;
    if (vec) {
        const int4 v = *reinterpret_cast<const int4*>(row + c);
        s0 = v.x; s1 = v.y; s2 = v.z; s3 = v.w;
    } else {
        s0 = row[c];
        if (c + 1 < n) s1 = row[c + 1];
        if (c + 2 < n) s2 = row[c + 2];
        if (c + 3 < n) s3 = row[c + 3];
    }
    const int sh = kCombBits * w;
    const unsigned f0 = (unsigned)(((unsigned long long)((long long)s0 + (long long)bias)) >> sh) & 7u;
    const unsigned f1 = (unsigned)(((unsigned long long)((long long)s1 + (long long)bias)) >> sh) & 7u;
    const unsigned f2 = (unsigned)(((unsigned long long)((long long)s2 + (long long)bias)) >> sh) & 7u;
    const unsigned f3 = (unsigned)(((unsigned long long)((long long)s3 + (long long)bias)) >> sh) & 7u;
    return f0 | (f1 << 3) | (f2 << 6) | (f3 << 9);
}

// Thread per (window, chain, row), rows fastest: one running sum over the chain's groups of four,
// skipping groups whose four digits are all zero (common in the top windows).  The table
// entry of the next step is requested from memory before the current addition starts.
#ifndef ZKB_COMB_MINBLOCKS
#define ZKB_COMB_MINBLOCKS 3
#endif
__global__ void __launch_bounds__(128, ZKB_COMB_MINBLOCKS) msm_comb_kernel(const G1Aff* __restrict__ table,
                                                                            const int32_t* __restrict__ scalars, CombShape sh,
                                                                            G1Jac* __restrict__ part) {
    const size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t total = (size_t)sh.W * sh.nseg * sh.m;
    if (t >= total) return;
    const size_t row = t % sh.m;
    const unsigned seg = (unsigned)((t / sh.m) % sh.nseg);
    // dense low windows first, the sparse top windows fill the tail of the launch
    const int w = (int)(t / (sh.m * sh.nseg));
    const unsigned long long bias = comb_bias(sh.W);
    const int32_t* srow = scalars + row * sh.n;
    // 16-byte loads of four scalars need n % 4 == 0 and an aligned matrix
    const bool vec = (sh.n & 3) == 0 && (reinterpret_cast<size_t>(scalars) & 15) == 0;
    size_t q = (size_t)seg * sh.qps;
    size_t q_end = q + sh.qps;
    if (q_end > sh.n_quads) q_end = sh.n_quads;
    // full groups can use the vector load; the ragged last group (n % 4 != 0) cannot
    unsigned idx = kCombZeroIdx;
    while (q < q_end && (idx = comb_index(srow, sh.n, q, w, bias, vec)) == kCombZeroIdx) ++q;
    G1Xyzz acc = xyzz_identity();
    while (q < q_end) {
        const G1Aff p = g1_aff_load(table + q * kCombEntries + idx);
        ++q;
        while (q < q_end && (idx = comb_index(srow, sh.n, q, w, bias, vec)) == kCombZeroIdx) ++q;
        if (q < q_end) {
            const char* nxt = reinterpret_cast<const char*>(table + q * kCombEntries + idx);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nxt));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nxt + 64));
        }
        acc = xyzz_add_mixed(acc, p);
    }
    g1_store(part + t, xyzz_to_jac(acc));
}

// Thread per (row, window): the chains of the window added up, times 8^w.  (Sixteen lanes per (row, window)
// with a shuffle tree were measured at 2.9 ms against 0.9 ms for this form on the 4096-row benchmark: the
// tree keeps whole warps busy for two sums.)
__global__ void __launch_bounds__(128) msm_comb_window_kernel(const G1Jac* __restrict__ part, CombShape sh, G1Jac* __restrict__ win) {
    const size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (t >= sh.m * (size_t)sh.W) return;
    const size_t row = t % sh.m;
    const int w = (int)(t / sh.m);
    G1Jac acc = g1_identity();
    for (unsigned sg = 0; sg < sh.nseg; ++sg) acc = g1_add(acc, g1_load(part + ((size_t)w * sh.nseg + sg) * sh.m + row));
    for (int d = 0; d < kCombBits * w; ++d) acc = g1_double(acc);
    g1_store(win + t, acc);
}

__global__ void __launch_bounds__(128) msm_comb_sum_kernel(const G1Jac* __restrict__ win, CombShape sh, G1Jac* __restrict__ out) {
    const size_t row = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (row >= sh.m) return;
    G1Jac acc = g1_load(win + row);
    for (int w = 1; w < sh.W; ++w) acc = g1_add(acc, g1_load(win + (size_t)w * sh.m + row));
    g1_store(out + row, acc);
}

// Products of field elements (unit of the two cost estimates below).
static double comb_cost(size_t m, size_t n, int W) {
    const double quads = (double)((n + 3) / 4);
    return (double)m * W * quads * 10.0 + quads * kCombEntries * 7.0;
}
static size_t comb_table_bytes(size_t n) { return ((n + 3) / 4) * (size_t)kCombEntries * sizeof(G1Aff); }

// Chains per (row, window): enough threads to fill the device, a whole number of waves
// when the chains are long enough to choose.
static unsigned comb_segments(size_t m, size_t n_quads, int W) {
    const size_t wave = (size_t)sm_count() * ZKB_COMB_MINBLOCKS * 128;
    unsigned best = 1;
    double best_eff = 0.0;
    for (unsigned nseg = 1; nseg <= 64; ++nseg) {
        if (nseg > 1 && n_quads / nseg < 48) break;
        const double waves = (double)(m * (size_t)W * nseg) / (double)wave;
        const double eff = waves / (double)(size_t)(waves + 0.999999);
        // prefer at least two waves worth of threads; among those, the fullest last wave
        const double score = (waves >= 2.0 ? 1.0 : waves / 2.0) * eff;
        if (score > best_eff + 1e-9) { best_eff = score; best = nseg; }
    }
    return best;
}

// The tables of one generator set: entry (q, i) = the combination of generators 4q..4q+3 with the four digits of i.
// They depend on the generators only, so a caller whose scalars are still on their way to the device can build them first.
static int comb_tables_build(const G1Aff* bases, size_t n, const G1Aff** table_out, Scratch& scratch, cudaStream_t s) {
    const size_t n_quads = (n + 3) / 4, n_pad = n_quads * 4, n_pairs = n_quads * 2;
    G1Aff* singles = scratch.get_n<G1Aff>(n_pad * 8);
    G1Aff* pairs = scratch.get_n<G1Aff>(n_pairs * 64);
    G1Aff* table = scratch.get_n<G1Aff>(n_quads * (size_t)kCombEntries);
    if (!singles || !pairs || !table) return ZKB_ERR_CUDA;
    ZKB_LAUNCH(comb_singles_kernel, div_up(n_pad, 128), 128, 0, s, bases, n, n_pad, singles);
    ZKB_LAUNCH(comb_pairs_kernel, div_up(n_pairs * 8, 128), 128, 0, s, singles, n_pairs, pairs);
    ZKB_LAUNCH(comb_quads_kernel, div_up(n_quads * 64, 128), 128, 0, s, pairs, n_quads, table);
    *table_out = table;
    return ZKB_OK;
}

// All rows through the tables of comb_tables_build.  scalars: int32 [m][n] with |s| within the range of W windows
// (comb_windows_for_max).
static int msm_comb_run(const G1Aff* table, size_t n, const int32_t* d_scalars, size_t m, int W,
                        G1Jac* d_out, Scratch& scratch, cudaStream_t s) {
    if (m == 0) return ZKB_OK;
    CombShape sh;
    sh.m = m; sh.n = n; sh.W = W;
    sh.n_quads = (n + 3) / 4;
    sh.nseg = comb_segments(m, sh.n_quads, W);
    sh.qps = (unsigned)((sh.n_quads + sh.nseg - 1) / sh.nseg);
    sh.nseg = (unsigned)((sh.n_quads + sh.qps - 1) / sh.qps);
    const size_t n_chains = (size_t)W * sh.nseg * m;
    G1Jac* part = scratch.get_n<G1Jac>(n_chains);
    G1Jac* win = scratch.get_n<G1Jac>((size_t)W * m);
    if (!part || !win) return ZKB_ERR_CUDA;
    if ((n_chains + 127) / 128 > 0x7fffffffull) return fail(ZKB_ERR_LIMIT, "commit: problem too large for one launch");
    ZKB_LAUNCH(msm_comb_kernel, div_up(n_chains, 128), 128, 0, s, table, d_scalars, sh, part);
    ZKB_LAUNCH(msm_comb_window_kernel, div_up(m * (size_t)W, 128), 128, 0, s, part, sh, win);
    ZKB_LAUNCH(msm_comb_sum_kernel, div_up(m, 128), 128, 0, s, win, sh, d_out);
    return ZKB_OK;
}

static int msm_comb_rows(const G1Aff* bases, size_t n, const int32_t* d_scalars, size_t m, int W,
                         G1Jac* d_out, Scratch& scratch, cudaStream_t s) {
    if (m == 0) return ZKB_OK;
    const G1Aff* table = nullptr;
    ZKB_TRY(comb_tables_build(bases, n, &table, scratch, s));
    return msm_comb_run(table, n, d_scalars, m, W, d_out, scratch, s);
}

}  // namespace zkb
