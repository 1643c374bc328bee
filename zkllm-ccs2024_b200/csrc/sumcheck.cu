// Sumcheck provers: zkip / zkFC::prove, tLookup::prove, multi-Hadamard and the
// legacy adjacent-pair sumchecks.
//
// The reference takes every challenge vector as an argument (or draws it up
// front), so all rounds of a proof are queued on the stream back to back: each
// round is ONE kernel that reads the current arrays once, accumulates the
// round-polynomial sums and writes the folded arrays; the grid-wide sums are
// finished by the last CTA of the same launch.  The host reads the sums once,
// after the last round, assembles the polynomials and replays the verifier
// checks (claim == p(0) + p(1)) that the reference makes between rounds.
#include "comm.cuh"
#include "frutil.cuh"
#include "hostfr.hpp"

#include <vector>

namespace zkb {

int partial_me_device(const Fr* d_a, size_t a_len, size_t other, size_t J, size_t window,
                      const zkb_fr_t* h_u, unsigned k, Fr* d_out, Scratch& scratch, cudaStream_t stream);

static constexpr unsigned kThreads = 256;
static constexpr unsigned kEqLoBits = 12;

static inline unsigned clog2(size_t n) {
    unsigned r = 0;
    if (n == 0) return 0;
    --n;
    while (n) { n >>= 1; ++r; }
    return r;
}
static inline Fr dev_fr(const hfr::H& h) {
    Fr r;
    memcpy(r.v, h.l, 32);
    return r;
}
static inline Fr dev_fr_mont(const zkb_fr_t& x) { return dev_fr(hfr::to_mont(hfr::load(x))); }

// eq weights for indices below 2^(kl+kh): lo table over the low kl bits, hi table
// (may be null) over the rest; both in Montgomery form.
struct EqTab {
    const Fr* lo;
    const Fr* hi;
    unsigned kl;
};

// The tables of every round of a proof in ONE launch: round r uses the k0 - r
// challenges that start at h_u[r * dstart] (dstart 0: a shrinking prefix, as in the
// MSB-first provers; dstart 1: a shrinking suffix, as in the legacy provers).
struct EqSeries {
    unsigned k0, rounds, dstart;
    unsigned lo_off[33], hi_off[33];   // entry offsets of each round's tables
};
__global__ void __launch_bounds__(256) eq_series_kernel(Challenges ch, EqSeries sr, Fr* __restrict__ lo_base, Fr* __restrict__ hi_base) {
    __shared__ Fr f1[32], f0[32];   // u_j * R and (1 - u_j) * R
    const unsigned r = blockIdx.y;
    const unsigned k = sr.k0 - r, start = r * sr.dstart;
    if (threadIdx.x < k) {
        const Fr um = to_mont<FrP>(ch.u[start + threadIdx.x]);
        f1[threadIdx.x] = um;
        f0[threadIdx.x] = fr_sub(fe_mont_one<FrP>(), um);
    }
    __syncthreads();
    const unsigned kl = k < kEqLoBits ? k : kEqLoBits, kh = k - kl;
    const size_t n_lo = (size_t)1 << kl, n_all = n_lo + (kh ? (size_t)1 << kh : 0);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_all; i += (size_t)gridDim.x * blockDim.x) {
        const bool high = i >= n_lo;
        const size_t idx = high ? i - n_lo : i;
        const unsigned nb = high ? kh : kl, b0 = high ? kl : 0;
        Fr acc = fe_mont_one<FrP>();
        for (unsigned j = 0; j < nb; ++j) acc = fr_mmul(acc, ((idx >> j) & 1) ? f1[b0 + j] : f0[b0 + j]);
        fr_store((high ? hi_base + sr.hi_off[r] : lo_base + sr.lo_off[r]) + idx, acc);
    }
}

static int make_eq_series(const zkb_fr_t* h_u, unsigned k0, unsigned rounds, unsigned dstart, EqTab* tabs,
                          Scratch& scratch, cudaStream_t s) {
    if (rounds == 0) return ZKB_OK;
    if (rounds > 33 || rounds > k0 + 1 || k0 > 32) return fail(ZKB_ERR_LIMIT, "eq tables: more than 32 variables");
    EqSeries sr;
    memset(&sr, 0, sizeof(sr));
    sr.k0 = k0; sr.rounds = rounds; sr.dstart = dstart;
    size_t lo_total = 0, hi_total = 0, max_entries = 0;
    for (unsigned r = 0; r < rounds; ++r) {
        const unsigned k = k0 - r, kl = k < kEqLoBits ? k : kEqLoBits, kh = k - kl;
        sr.lo_off[r] = (unsigned)lo_total;
        sr.hi_off[r] = (unsigned)hi_total;
        lo_total += (size_t)1 << kl;
        if (kh) hi_total += (size_t)1 << kh;
        const size_t e = ((size_t)1 << kl) + (kh ? (size_t)1 << kh : 0);
        if (e > max_entries) max_entries = e;
    }
    if (hi_total > 0xffffffffull) return fail(ZKB_ERR_LIMIT, "eq tables: too large");
    Fr* lo = scratch.get_n<Fr>(lo_total);
    Fr* hi = hi_total ? scratch.get_n<Fr>(hi_total) : nullptr;
    if (!lo || (hi_total && !hi)) return ZKB_ERR_CUDA;
    Challenges ch;
    memset(&ch, 0, sizeof(ch));
    for (unsigned j = 0; j < k0; ++j) memcpy(ch.u[j].v, h_u[j].val, 32);
    unsigned gx = grid_for(max_entries, 256, 2);
    ZKB_LAUNCH(eq_series_kernel, dim3(gx, rounds), 256, 0, s, ch, sr, lo, hi);
    for (unsigned r = 0; r < rounds; ++r) {
        const unsigned k = k0 - r, kl = k < kEqLoBits ? k : kEqLoBits, kh = k - kl;
        tabs[r].lo = lo + sr.lo_off[r];
        tabs[r].hi = kh ? hi + sr.hi_off[r] : nullptr;
        tabs[r].kl = kl;
    }
    return ZKB_OK;
}

// Work split of the eq-weighted round kernels: a CTA walks "pieces" of
// blockDim.x * R consecutive indices (R a power of two, at most 16, so a piece
// never straddles a 4096-entry chunk of the low table and the high-table
// factor is applied once per piece).  R shrinks for small arrays so that
// there are enough pieces to occupy the GPU.
static void pieces_for(size_t count, unsigned* R, unsigned* grid) {
    unsigned r = 16;
    const size_t want = (size_t)sm_count() * 2;
    while (r > 1 && (count + (size_t)kThreads * r - 1) / ((size_t)kThreads * r) < want) r >>= 1;
    const size_t npieces = (count + (size_t)kThreads * r - 1) / ((size_t)kThreads * r);
    const size_t cap = (size_t)sm_count() * 4;
    *R = r;
    *grid = (unsigned)(npieces < 1 ? 1 : (npieces < cap ? npieces : cap));
}

// ---------------------------------------------------------------------------
// zkip round: pairs (g, g + half); sums of c0, c1, c2; folded outputs.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) zkip_round_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b,
                                                               size_t n_in, size_t half, Fr v_mont,
                                                               Fr* __restrict__ na, Fr* __restrict__ nb,
                                                               Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[3];
    acc[0] = acc[1] = acc[2] = fr_zero();
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < half; g += (size_t)gridDim.x * blockDim.x) {
        const Fr a0 = g < n_in ? fr_load(a + g) : fr_zero();
        const Fr b0 = g < n_in ? fr_load(b + g) : fr_zero();
        const Fr a1 = g + half < n_in ? fr_load(a + g + half) : fr_zero();
        const Fr b1 = g + half < n_in ? fr_load(b + g + half) : fr_zero();
        const Fr da = fr_sub(a1, a0), db = fr_sub(b1, b0);
        const Fr t0 = fr_mmul(a0, b0), t2 = fr_mmul(da, db);
        // a0*db + b0*da = a1*b1 - a0*b0 - da*db
        const Fr t1 = fr_sub(fr_sub(fr_mmul(a1, b1), t0), t2);
        acc[0] = fr_add(acc[0], t0);
        acc[1] = fr_add(acc[1], t1);
        acc[2] = fr_add(acc[2], t2);
        fr_store(na + g, fr_add(a0, fr_mmul(v_mont, da)));
        fr_store(nb + g, fr_add(b0, fr_mmul(v_mont, db)));
    }
    grid_sum_finish<3>(acc, partial, ticket, out, 0x7u, red);
}

// One round of zkip_stacked (zkfc.cu:153-228): A and B are [num, D]; the round pairs head h with head
// h + half_heads (zero past the last head), weights the three coefficient sums by eq(u_; h) over the lower
// heads and folds the head axis with v.  One pass over A and B instead of the reference's two kernels,
// three D-long fold passes and three sums.  `eq` covers the half_heads lower heads (lo/hi split as elsewhere).
__global__ void __launch_bounds__(kThreads) zkip_stacked_round_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b, size_t n_in,
                                                                       size_t half, size_t D, Fr v_mont, EqTab eq,
                                                                       Fr* __restrict__ na, Fr* __restrict__ nb,
                                                                       Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[3];
    acc[0] = acc[1] = acc[2] = fr_zero();
    const size_t lmask = ((size_t)1 << eq.kl) - 1;
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < half; g += (size_t)gridDim.x * blockDim.x) {
        const size_t head = g / D;
        Fr e = fr_load(eq.lo + (head & lmask));
        if (eq.hi) e = fr_mmul(e, fr_load(eq.hi + (head >> eq.kl)));      // (lo R)(hi R)/R = e R
        const Fr a0 = fr_load(a + g), b0 = fr_load(b + g);
        const Fr a1 = g + half < n_in ? fr_load(a + g + half) : fr_zero();
        const Fr b1 = g + half < n_in ? fr_load(b + g + half) : fr_zero();
        const Fr da = fr_sub(a1, a0), db = fr_sub(b1, b0);
        const Fr e0 = fr_mmul(a0, e), e1 = fr_mmul(da, e);
        const Fr t0 = fr_mmul(e0, b0), t2 = fr_mmul(e1, db);
        const Fr t1 = fr_sub(fr_sub(fr_mmul(fr_add(e0, e1), fr_add(b0, db)), t0), t2);
        acc[0] = fr_add(acc[0], t0);
        acc[1] = fr_add(acc[1], t1);
        acc[2] = fr_add(acc[2], t2);
        fr_store(na + g, fr_add(a0, fr_mmul(v_mont, da)));
        fr_store(nb + g, fr_add(b0, fr_mmul(v_mont, db)));
    }
    grid_sum_finish<3>(acc, partial, ticket, out, 0x7u, red);
}

// The last rounds of zkip in ONE launch of one CTA: from kZkipTailHalf pairs down (above that one SM is too slow),
// a round is a few microseconds of work and a separate launch each would cost
// more than the arithmetic.  `vs` holds the challenges of these rounds in round
// order (Montgomery form); wa/wb are two ping-pong buffers of `half` entries each.
static constexpr size_t kZkipTailHalf = 512;
static constexpr unsigned kZkipTailThreads = 512;

// A sum of up to 2^32 field elements as a plain 288-bit integer: adding is one carry chain, the
// reduction modulo r happens once per sum instead of once per addition.
struct Wide9 { uint32_t l[9]; };
ZKB_DEV void wide_zero(Wide9& w) {
#pragma unroll
    for (int i = 0; i < 9; ++i) w.l[i] = 0u;
}
ZKB_DEV void wide_add_fr(Wide9& w, const Fr& a) {
    ptx_add_cc(w.l[0], a.v[0]);
#pragma unroll
    for (int i = 1; i < 8; ++i) ptx_addc_cc(w.l[i], a.v[i]);
    ptx_addc(w.l[8], 0u);
}
ZKB_DEV void wide_add(Wide9& w, const Wide9& o) {
    ptx_add_cc(w.l[0], o.l[0]);
#pragma unroll
    for (int i = 1; i < 8; ++i) ptx_addc_cc(w.l[i], o.l[i]);
    ptx_addc(w.l[8], o.l[8]);
}
ZKB_DEV Wide9 wide_shfl_down(const Wide9& w, int off) {
    Wide9 o;
#pragma unroll
    for (int i = 0; i < 9; ++i) o.l[i] = __shfl_down_sync(0xffffffffu, w.l[i], off);
    return o;
}
// (w * R) mod r for w = lo + hi 2^256: the sum of raw Montgomery products (each carrying 1/R) as the
// true field element.
ZKB_DEV Fr wide_fix(const Wide9& w) {
    Fr lo, hi = fr_zero();
#pragma unroll
    for (int i = 0; i < 8; ++i) lo.v[i] = w.l[i];
    fe_final_sub(lo);   // 2^256 < 3r: two conditional subtractions make lo canonical
    fe_final_sub(lo);
    hi.v[0] = w.l[8];
    const Fr r2 = fe_r2<FrP>();
    // lo R + hi 2^256 R = lo R + hi R^2
    return fr_add(fr_mmul(lo, r2), fr_mmul(fr_mmul(hi, r2), r2));
}

__global__ void __launch_bounds__(kZkipTailThreads) zkip_tail_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b, size_t n_in,
                                                                      size_t half, Challenges vs, unsigned rounds,
                                                                      Fr* __restrict__ wa, Fr* __restrict__ wb, Fr* __restrict__ out) {
    __shared__ Wide9 stage[3][kZkipTailThreads / 32];
    const size_t stride = half;
    const Fr* ca = a;
    const Fr* cb = b;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (unsigned r = 0; r < rounds; ++r) {
        Fr* oa = wa + (r & 1) * stride;
        Fr* ob = wb + (r & 1) * stride;
        const Fr v_mont = vs.u[r];
        // warps that hold a pair of this round; the others only meet the barriers
        const unsigned active_warps = (unsigned)((half + 31) / 32 < kZkipTailThreads / 32 ? (half + 31) / 32 : kZkipTailThreads / 32);
        if ((unsigned)warp < active_warps) {
            Wide9 acc[3];
            wide_zero(acc[0]); wide_zero(acc[1]); wide_zero(acc[2]);
            for (size_t g = threadIdx.x; g < half; g += (size_t)active_warps * 32) {
                const Fr a0 = g < n_in ? fr_load(ca + g) : fr_zero();
                const Fr b0 = g < n_in ? fr_load(cb + g) : fr_zero();
                const Fr a1 = g + half < n_in ? fr_load(ca + g + half) : fr_zero();
                const Fr b1 = g + half < n_in ? fr_load(cb + g + half) : fr_zero();
                const Fr da = fr_sub(a1, a0), db = fr_sub(b1, b0);
                const Fr t0 = fr_mmul(a0, b0), t2 = fr_mmul(da, db);
                const Fr t1 = fr_sub(fr_sub(fr_mmul(a1, b1), t0), t2);
                wide_add_fr(acc[0], t0);
                wide_add_fr(acc[1], t1);
                wide_add_fr(acc[2], t2);
                fr_store(oa + g, fr_add(a0, fr_mmul(v_mont, da)));
                fr_store(ob + g, fr_add(b0, fr_mmul(v_mont, db)));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
                for (int q = 0; q < 3; ++q) wide_add(acc[q], wide_shfl_down(acc[q], off));
            }
            if (lane == 0) {
#pragma unroll
                for (int q = 0; q < 3; ++q) stage[q][warp] = acc[q];
            }
        }
        __syncthreads();                       // also orders this round's stores before the next round's loads
        if (threadIdx.x < 3) {
            Wide9 tot = stage[threadIdx.x][0];
            for (unsigned w = 1; w < active_warps; ++w) wide_add(tot, stage[threadIdx.x][w]);
            fr_store(out + 3 * r + threadIdx.x, wide_fix(tot));
        }
        __syncthreads();
        ca = oa;
        cb = ob;
        n_in = half;
        half >>= 1;
    }
}

// Queues the first `run` of the k rounds of zkip on `s` (round r uses h_u[k - 1 - r]).
// d_polys receives 3 Fr per round.  fin_a / fin_b (optional) receive device pointers
// to the arrays as folded by the last round queued (length 2^(ceilLog2(n) - run)); the
// protocol itself does not need them after its last round.
static int zkip_device(const Fr* d_a, const Fr* d_b, size_t n, const zkb_fr_t* h_u, unsigned k, unsigned run,
                       Fr* d_polys, Scratch& scratch, cudaStream_t s, const Fr** fin_a = nullptr, const Fr** fin_b = nullptr) {
    if (fin_a) *fin_a = d_a;
    if (fin_b) *fin_b = d_b;
    if (run == 0) return ZKB_OK;
    const unsigned kn = clog2(n);
    if (k > kn) return fail(ZKB_ERR_DIM, "zkip: more challenges than variables");
    if (run > k) return fail(ZKB_ERR_ARG, "zkip: more rounds than challenges");
    size_t half = ((size_t)1 << kn) >> 1;
    const Fr* ca = d_a;
    const Fr* cb = d_b;
    size_t n_in = n;
    unsigned r = 0;
    if (half > kZkipTailHalf) {
        Fr* buf[2][2];
        for (int i = 0; i < 2; ++i)
            for (int j = 0; j < 2; ++j) {
                buf[i][j] = scratch.get_n<Fr>(half >> i ? half >> i : 1);
                if (!buf[i][j]) return ZKB_ERR_CUDA;
            }
        const unsigned max_grid = grid_for(half, kThreads, 4);
        Fr* partial = scratch.get_n<Fr>((size_t)max_grid * 3);
        unsigned* ticket = scratch.get_n<unsigned>(4);
        if (!partial || !ticket) return ZKB_ERR_CUDA;
        ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
        for (; r < run && half > kZkipTailHalf; ++r) {
            const Fr v = dev_fr_mont(h_u[k - 1 - r]);
            Fr* oa = buf[r & 1][0];
            Fr* ob = buf[r & 1][1];
            ZKB_LAUNCH(zkip_round_kernel, grid_for(half, kThreads, 4), kThreads, 0, s,
                       ca, cb, n_in, half, v, oa, ob, partial, ticket, d_polys + 3 * r);
            ca = oa; cb = ob;
            n_in = half;
            half >>= 1;
        }
    }
    if (r < run) {
        const unsigned rounds = run - r;   // at most 10: half <= 512 here
        Challenges vs;
        memset(&vs, 0, sizeof(vs));
        for (unsigned t = 0; t < rounds; ++t) vs.u[t] = dev_fr_mont(h_u[k - 1 - (r + t)]);
        Fr* wa = scratch.get_n<Fr>(2 * half);
        Fr* wb = scratch.get_n<Fr>(2 * half);
        if (!wa || !wb) return ZKB_ERR_CUDA;
        ZKB_LAUNCH(zkip_tail_kernel, 1, kZkipTailThreads, 0, s, ca, cb, n_in, half, vs, rounds, wa, wb, d_polys + 3 * r);
        // the tail's round t writes to the half of the ping-pong pair with index t & 1
        ca = wa + ((rounds - 1) & 1) * half;
        cb = wb + ((rounds - 1) & 1) * half;
    }
    if (fin_a) *fin_a = ca;
    if (fin_b) *fin_b = cb;
    return ZKB_OK;
}

// Host replay of the verifier checks of zkip (zkfc.cu:140-151).
static int zkip_verify(const zkb_fr_t* h_claim, const zkb_fr_t* h_u, unsigned k, const zkb_fr_t* polys, zkb_fr_t* h_final) {
    hfr::H claim = hfr::load(*h_claim);
    for (unsigned r = 0; r < k; ++r) {
        hfr::H c[3] = {hfr::load(polys[3 * r]), hfr::load(polys[3 * r + 1]), hfr::load(polys[3 * r + 2])};
        hfr::H p0 = c[0];
        hfr::H p1 = hfr::add(hfr::add(c[0], c[1]), c[2]);
        if (!hfr::eq(claim, hfr::add(p0, p1))) return fail(ZKB_ERR_VERIFY, "claim != p(0) + p(1)");
        claim = hfr::poly_eval(c, 3, hfr::load(h_u[k - 1 - r]));
    }
    *h_final = hfr::store(claim);
    return ZKB_OK;
}

// ---------------------------------------------------------------------------
// tLookup rounds
// ---------------------------------------------------------------------------
// Phase-1 round on (A, S) of size 2*half (tlookup.cu:74-109, 184-200).
// sums: [0..2] eq-weighted coefficients of (A0 + A1 t)(S0 + beta + S1 t) (without
// the alpha factor, applied on the host), [3] sum A0, [4] sum A1.
// Resident CTAs per SM asked of the compiler for the two phase-1 kernels (register cap 65536 / (256 * this)).
// Measured on the 2^23-value proof: 2 (128 registers, a few hundred bytes of spills) 405 + 856 us for the first and the
// six later rounds against 544 + 904 us with 1 (218 / 174 registers, 8 warps per SM).
#ifndef ZKB_TL_MINBLOCKS
#define ZKB_TL_MINBLOCKS 2
#endif
__global__ void __launch_bounds__(kThreads, ZKB_TL_MINBLOCKS) tl_phase1_kernel(const Fr* __restrict__ A, const Fr* __restrict__ S, size_t half,
                                                              Fr beta, Fr v_mont, EqTab eq, unsigned R,
                                                              Fr* __restrict__ nA, Fr* __restrict__ nS,
                                                              Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[5];
#pragma unroll
    for (int i = 0; i < 5; ++i) acc[i] = fr_zero();
    const size_t lmask = ((size_t)1 << eq.kl) - 1;
    const size_t piece = (size_t)blockDim.x * R;          // never straddles a chunk of the low table
    const size_t npieces = (half + piece - 1) / piece;
    for (size_t c = blockIdx.x; c < npieces; c += gridDim.x) {
        Fr q0 = fr_zero(), q1 = fr_zero(), q2 = fr_zero();
        const size_t base = c * piece;
        for (size_t jj = threadIdx.x; jj < piece && base + jj < half; jj += blockDim.x) {
            const size_t j = (base + jj) & lmask;
            const size_t i = base + jj;
            const Fr a0 = fr_load(A + i), a1 = fr_load(A + i + half);
            const Fr s0 = fr_load(S + i), s1 = fr_load(S + i + half);
            const Fr e = fr_load(eq.lo + j);
            const Fr c01 = fr_sub(a1, a0), c10 = fr_add(s0, beta), c11 = fr_sub(s1, s0);
            const Fr e00 = fr_mmul(a0, e), e01 = fr_mmul(c01, e);
            const Fr t0 = fr_mmul(e00, c10), t2 = fr_mmul(e01, c11);
            const Fr t1 = fr_sub(fr_sub(fr_mmul(fr_add(e00, e01), fr_add(c10, c11)), t0), t2);
            q0 = fr_add(q0, t0); q1 = fr_add(q1, t1); q2 = fr_add(q2, t2);
            acc[3] = fr_add(acc[3], a0);
            acc[4] = fr_add(acc[4], c01);
            fr_store(nA + i, fr_add(a0, fr_mmul(v_mont, c01)));
            fr_store(nS + i, fr_add(s0, fr_mmul(v_mont, c11)));
        }
        if (eq.hi) {
            const Fr eh = fr_load(eq.hi + (base >> eq.kl));
            q0 = fr_mmul(q0, eh); q1 = fr_mmul(q1, eh); q2 = fr_mmul(q2, eh);
        }
        acc[0] = fr_add(acc[0], q0); acc[1] = fr_add(acc[1], q1); acc[2] = fr_add(acc[2], q2);
    }
    grid_sum_finish<5>(acc, partial, ticket, out, 0x7u, red);
}

// 1 / (s + beta) for a value the caller says sits at table index k: B[k] when T[k] == s (B holds the
// inverses of the table), else the value's own inversion - the same field element either way, zero
// mapped to zero (tlookup_inv_kernel, tlookup.cu:50-62).
ZKB_DEV Fr tl_inverse_at(const Fr& s, uint32_t k, const Fr* __restrict__ T, const Fr* __restrict__ Bv, size_t N, const Fr& beta) {
    if (k < N && fe_eq(fr_load(T + k), s)) return fr_load(Bv + k);
    const Fr x = fr_add(s, beta);
    if (fe_is_zero(x)) return x;
    Fr one = fr_zero();
    one.v[0] = 1u;
    // x read as the Montgomery form of x / R: the inverse comes back as R^2 / x
    return fr_mmul(fr_mmul(mont_inv<FrP>(x), one), one);
}

// First phase-1 round with A = 1 / (S + beta) formed on the fly from the table's inverses, so the
// D-element array A is neither computed by D inversions nor written and read back.  Same five
// sums and the same folded arrays as tl_phase1_kernel on (A, S).  Where both inverses of a pair
// are non-zero, A0 (S0 + beta) = A1 (S1 + beta) = 1 exactly, which turns the three weighted
// coefficients into
//     t0 = e,    t2 = e (A1 - A0)(S1 - S0),    t1 = -t2,
// one field product and one product by the difference S1 - S0 - a small integer for fixed-point
// data, accumulated unreduced (LazyDot).  A pair with a zero inverse takes the general formulas.
__global__ void __launch_bounds__(kThreads, ZKB_TL_MINBLOCKS) tl_phase1_first_kernel(const Fr* __restrict__ S, const uint32_t* __restrict__ idx,
                                                                    const Fr* __restrict__ T, const Fr* __restrict__ Bv, size_t N,
                                                                    size_t half, Fr beta, Fr v_mont, EqTab eq, unsigned R,
                                                                    Fr* __restrict__ nA, Fr* __restrict__ nS,
                                                                    Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[5];
#pragma unroll
    for (int i = 0; i < 5; ++i) acc[i] = fr_zero();
    Fr one = fr_zero();
    one.v[0] = 1u;
    const size_t lmask = ((size_t)1 << eq.kl) - 1;
    const size_t piece = (size_t)blockDim.x * R;          // never straddles a chunk of the low table
    const size_t npieces = (half + piece - 1) / piece;
    for (size_t c = blockIdx.x; c < npieces; c += gridDim.x) {
        Fr esum = fr_zero();                               // sum of the weights e R of the regular pairs
        LazyDot lazy;                                      // sum of (S1 - S0) * e (A1 - A0), carries 1/R after finish()
        lazy.init();
        const size_t base = c * piece;
        for (size_t jj = threadIdx.x; jj < piece && base + jj < half; jj += blockDim.x) {
            const size_t j = (base + jj) & lmask;
            const size_t i = base + jj;
            const Fr s0 = fr_load(S + i), s1 = fr_load(S + i + half);
            const Fr a0 = tl_inverse_at(s0, idx[i], T, Bv, N, beta);
            const Fr a1 = tl_inverse_at(s1, idx[i + half], T, Bv, N, beta);
            const Fr e = fr_load(eq.lo + j);
            const Fr c01 = fr_sub(a1, a0), c11 = fr_sub(s1, s0);
            const Fr e01 = fr_mmul(c01, e);
            if (!fe_is_zero(a0) && !fe_is_zero(a1)) {
                esum = fr_add(esum, e);
                lazy.add(c11, e01);
            } else {
                // rare (S + beta = 0 somewhere in the pair): the general formulas, weighted in full at once so that
                // the common path carries no accumulators for them
                const Fr c10 = fr_add(s0, beta);
                const Fr e00 = fr_mmul(a0, e);
                Fr t0 = fr_mmul(e00, c10), t2 = fr_mmul(e01, c11);
                Fr t1 = fr_sub(fr_sub(fr_mmul(fr_add(e00, e01), fr_add(c10, c11)), t0), t2);
                if (eq.hi) {
                    const Fr eh = fr_load(eq.hi + (base >> eq.kl));
                    t0 = fr_mmul(t0, eh); t1 = fr_mmul(t1, eh); t2 = fr_mmul(t2, eh);
                }
                acc[0] = fr_add(acc[0], t0); acc[1] = fr_add(acc[1], t1); acc[2] = fr_add(acc[2], t2);
            }
            acc[3] = fr_add(acc[3], a0);
            acc[4] = fr_add(acc[4], c01);
            fr_store(nA + i, fr_add(a0, fr_mmul(v_mont, c01)));
            fr_store(nS + i, fr_add(s0, fr_mmul(v_mont, c11)));
        }
        // e R -> e / R, the scale of the other weighted terms (fixed by R^2 after the grid sum)
        Fr q0 = fr_mmul(fr_mmul(esum, one), one);
        Fr q2 = lazy.finish();
        if (eq.hi) {
            const Fr eh = fr_load(eq.hi + (base >> eq.kl));
            q0 = fr_mmul(q0, eh); q2 = fr_mmul(q2, eh);
        }
        acc[0] = fr_add(acc[0], q0); acc[1] = fr_sub(acc[1], q2); acc[2] = fr_add(acc[2], q2);
    }
    grid_sum_finish<5>(acc, partial, ticket, out, 0x7u, red);
}

// One pair (i, i + half) of a phase-2 round: the eq-weighted terms go to q[0..5], the
// plain ones to acc[6..10]; the five folded values are stored.
ZKB_DEV void tl_phase2_pair(const Fr* __restrict__ A, const Fr* __restrict__ S, const Fr* __restrict__ Bv, const Fr* __restrict__ T,
                            const Fr* __restrict__ m, size_t i, size_t half, const Fr& beta, const Fr& v_mont, const Fr& e,
                            Fr* __restrict__ nA, Fr* __restrict__ nS, Fr* __restrict__ nB, Fr* __restrict__ nT, Fr* __restrict__ nm,
                            Fr (&q)[6], Fr (&acc)[11]) {
    {
        const Fr a0 = fr_load(A + i), a1 = fr_load(A + i + half);
        const Fr s0 = fr_load(S + i), s1 = fr_load(S + i + half);
        const Fr c01 = fr_sub(a1, a0), c10 = fr_add(s0, beta), c11 = fr_sub(s1, s0);
        const Fr e00 = fr_mmul(a0, e), e01 = fr_mmul(c01, e);
        const Fr t0 = fr_mmul(e00, c10), t2 = fr_mmul(e01, c11);
        const Fr t1 = fr_sub(fr_sub(fr_mmul(fr_add(e00, e01), fr_add(c10, c11)), t0), t2);
        q[0] = fr_add(q[0], t0); q[1] = fr_add(q[1], t1); q[2] = fr_add(q[2], t2);
        acc[6] = fr_add(acc[6], a0);
        acc[7] = fr_add(acc[7], c01);
        fr_store(nA + i, fr_add(a0, fr_mmul(v_mont, c01)));
        fr_store(nS + i, fr_add(s0, fr_mmul(v_mont, c11)));
    }
    {
        const Fr b0 = fr_load(Bv + i), b1 = fr_load(Bv + i + half);
        const Fr t0_ = fr_load(T + i), t1_ = fr_load(T + i + half);
        const Fr m0 = fr_load(m + i), m1f = fr_load(m + i + half);
        const Fr c01 = fr_sub(b1, b0), c10 = fr_add(t0_, beta), c11 = fr_sub(t1_, t0_);
        const Fr e00 = fr_mmul(b0, e), e01 = fr_mmul(c01, e);
        const Fr t0 = fr_mmul(e00, c10), t2 = fr_mmul(e01, c11);
        const Fr t1 = fr_sub(fr_sub(fr_mmul(fr_add(e00, e01), fr_add(c10, c11)), t0), t2);
        q[3] = fr_add(q[3], t0); q[4] = fr_add(q[4], t1); q[5] = fr_add(q[5], t2);
        const Fr m1 = fr_sub(m1f, m0);
        const Fr d0 = fr_mmul(m0, b0), d2 = fr_mmul(m1, c01);
        const Fr d1 = fr_sub(fr_sub(fr_mmul(m1f, b1), d0), d2);
        acc[8] = fr_add(acc[8], d0); acc[9] = fr_add(acc[9], d1); acc[10] = fr_add(acc[10], d2);
        fr_store(nB + i, fr_add(b0, fr_mmul(v_mont, c01)));
        fr_store(nT + i, fr_add(t0_, fr_mmul(v_mont, c11)));
        fr_store(nm + i, fr_add(m0, fr_mmul(v_mont, m1)));
    }
}

// The last phase-2 rounds (at most kTlTailHalf pairs) in ONE launch of one CTA of 128
// threads, like zkip_tail_kernel.  Round t reads `cur`, writes the ping-pong set `nxt[t & 1]`
// and uses the eq table lo[t] (these rounds have at most 7 variables: no high table).
static constexpr size_t kTlTailHalf = 128;
static constexpr unsigned kTlTailRounds = 8;
struct TlTail {
    const Fr* cur[5];                 // A, S, B, T, m as the first tail round finds them
    Fr* nxt[2][5];                    // outputs of even / odd tail rounds
    const Fr* lo[kTlTailRounds];      // eq tables per round (Montgomery form)
    Fr v[kTlTailRounds];              // challenges per round (Montgomery form)
};
__global__ void __launch_bounds__(128) tl_phase2_tail_kernel(TlTail tt, size_t half, Fr beta, unsigned rounds, Fr* __restrict__ out) {
    __shared__ Fr stage[11][4];
    const Fr* in[5];
#pragma unroll
    for (int a = 0; a < 5; ++a) in[a] = tt.cur[a];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (unsigned t = 0; t < rounds; ++t) {
        Fr acc[11], q[6];
#pragma unroll
        for (int i = 0; i < 11; ++i) acc[i] = fr_zero();
#pragma unroll
        for (int i = 0; i < 6; ++i) q[i] = fr_zero();
        Fr* const* o = tt.nxt[t & 1];
        for (size_t i = threadIdx.x; i < half; i += blockDim.x)
            tl_phase2_pair(in[0], in[1], in[2], in[3], in[4], i, half, beta, tt.v[t], fr_load(tt.lo[t] + i), o[0], o[1], o[2], o[3], o[4],
                           q, acc);
#pragma unroll
        for (int i = 0; i < 6; ++i) acc[i] = q[i];
#pragma unroll
        for (int i = 0; i < 11; ++i) {
            acc[i] = warp_sum(acc[i]);
            if (lane == 0) stage[i][warp] = acc[i];
        }
        __syncthreads();                 // also orders this round's stores before the next round's loads
        if (threadIdx.x < 11) {
            Fr v = fr_add(fr_add(stage[threadIdx.x][0], stage[threadIdx.x][1]), fr_add(stage[threadIdx.x][2], stage[threadIdx.x][3]));
            if ((0x73Fu >> threadIdx.x) & 1u) v = fr_mmul(v, fe_r2<FrP>());   // sums of raw Montgomery products
            fr_store(out + 11 * (size_t)t + threadIdx.x, v);
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < 5; ++a) in[a] = o[a];
        half >>= 1;
    }
}

// Phase-2 round on (A, S, B, T, m) of size 2*half (tlookup.cu:161-279).
// sums: [0..2] eq-weighted (A,S) coefficients, [3..5] eq-weighted (B,T)
// coefficients, [6] sum A0, [7] sum A1, [8..10] coefficients of (m0 + m1 t)(B0 + B1 t).
__global__ void __launch_bounds__(kThreads) tl_phase2_kernel(const Fr* __restrict__ A, const Fr* __restrict__ S,
                                                              const Fr* __restrict__ Bv, const Fr* __restrict__ T,
                                                              const Fr* __restrict__ m, size_t half,
                                                              Fr beta, Fr v_mont, EqTab eq, unsigned R,
                                                              Fr* __restrict__ nA, Fr* __restrict__ nS, Fr* __restrict__ nB,
                                                              Fr* __restrict__ nT, Fr* __restrict__ nm,
                                                              Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[11];
#pragma unroll
    for (int i = 0; i < 11; ++i) acc[i] = fr_zero();
    const size_t lmask = ((size_t)1 << eq.kl) - 1;
    const size_t piece = (size_t)blockDim.x * R;          // never straddles a chunk of the low table
    const size_t npieces = (half + piece - 1) / piece;
    for (size_t c = blockIdx.x; c < npieces; c += gridDim.x) {
        Fr q[6];
#pragma unroll
        for (int i = 0; i < 6; ++i) q[i] = fr_zero();
        const size_t base = c * piece;
        for (size_t jj = threadIdx.x; jj < piece && base + jj < half; jj += blockDim.x) {
            const size_t j = (base + jj) & lmask;
            const size_t i = base + jj;
            tl_phase2_pair(A, S, Bv, T, m, i, half, beta, v_mont, fr_load(eq.lo + j), nA, nS, nB, nT, nm, q, acc);
        }
        if (eq.hi) {
            const Fr eh = fr_load(eq.hi + (base >> eq.kl));
#pragma unroll
            for (int t = 0; t < 6; ++t) q[t] = fr_mmul(q[t], eh);
        }
#pragma unroll
        for (int t = 0; t < 6; ++t) acc[t] = fr_add(acc[t], q[t]);
    }
    grid_sum_finish<11>(acc, partial, ticket, out, 0x73Fu, red);
}

// out[0] = sum a[i]*b[i].  fix = 1 when both operands are standard-form tensor
// values, 0 when b is a Montgomery-form table.
__global__ void __launch_bounds__(kThreads) fr_dot_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b, size_t n,
                                                           Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out,
                                                           unsigned fix) {
    __shared__ Fr red[32];
    Fr acc[1];
    acc[0] = fr_zero();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        acc[0] = fr_add(acc[0], fr_mmul(fr_load(a + i), fr_load(b + i)));
    grid_sum_finish<1>(acc, partial, ticket, out, fix, red);
}

// Multiplicities: counts[k] = how many indices equal k.  Lanes of a warp that hold the same index add once for all of
// them: padded tensors and activations that are mostly zero put millions of entries into one table slot, and that many
// atomics on one address take milliseconds (4.5 ms for 2^25 entries with 11 million equal ones; 0.3 ms this way).
__global__ void tl_count_kernel(const uint32_t* __restrict__ idx, size_t D, size_t N, uint32_t* __restrict__ counts) {
    const unsigned lane = threadIdx.x & 31u;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t base = blockIdx.x * (size_t)blockDim.x + (threadIdx.x - lane); base < D; base += stride) {   // warp-uniform
        const size_t i = base + lane;
        uint32_t k = 0xffffffffu;
        if (i < D) {
            k = idx[i];
            if (k >= N) k = 0xffffffffu;
        }
        const unsigned same = __match_any_sync(0xffffffffu, k);
        if (k != 0xffffffffu && lane == (unsigned)(__ffs((int)same) - 1)) atomicAdd(counts + k, (uint32_t)__popc(same));
    }
}
__global__ void tl_counts_to_fr_kernel(const uint32_t* __restrict__ counts, size_t N, Fr* __restrict__ m) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < N; i += (size_t)gridDim.x * blockDim.x)
        fr_store(m + i, fr_from_u64(counts[i]));
}
__global__ void tl_range_indices_kernel(const Fr* __restrict__ vals, Fr low, uint32_t* __restrict__ idx, size_t D) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < D; i += (size_t)gridDim.x * blockDim.x)
        idx[i] = fr_sub(fr_load(vals + i), low).v[0];
}
__global__ void tl_range_table_kernel(int low, size_t len, size_t size, Fr* __restrict__ table) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < size; i += (size_t)gridDim.x * blockDim.x) {
        const int val = (i < len) ? static_cast<int>(i) + low : static_cast<int>(len) + low - 1;
        fr_store(table + i, fr_from_i64(val));
    }
}

// ---------------------------------------------------------------------------
// multi-Hadamard round (proof.cu:172-241): K arrays of size 2*half.
// sums: K+1 eq-weighted coefficients of prod_k (X0_k + X1_k t).
// ---------------------------------------------------------------------------
static constexpr int kMaxHadamard = 6;
struct HadamardPtrs {
    const Fr* in[kMaxHadamard];
    Fr* out[kMaxHadamard];
};
template <int K>
__global__ void __launch_bounds__(kThreads) hadamard_round_kernel(HadamardPtrs p, size_t half, Fr v_mont, EqTab eq, unsigned R,
                                                                   Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[K + 1];
#pragma unroll
    for (int i = 0; i <= K; ++i) acc[i] = fr_zero();
    const size_t lmask = ((size_t)1 << eq.kl) - 1;
    const size_t piece = (size_t)blockDim.x * R;          // never straddles a chunk of the low table
    const size_t npieces = (half + piece - 1) / piece;
    for (size_t c = blockIdx.x; c < npieces; c += gridDim.x) {
        Fr q[K + 1];
#pragma unroll
        for (int i = 0; i <= K; ++i) q[i] = fr_zero();
        const size_t base = c * piece;
        for (size_t jj = threadIdx.x; jj < piece && base + jj < half; jj += blockDim.x) {
            const size_t j = (base + jj) & lmask;
            const size_t i = base + jj;
            // Running product polynomial.  It starts as e*R (Montgomery form); the
            // first multiplication by a standard-form value gives e*x exactly and
            // every further one adds a factor 1/R, removed after the grid sum.
            Fr poly[K + 1];
            poly[0] = fr_load(eq.lo + j);
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const Fr x0 = fr_load(p.in[k] + i), x1f = fr_load(p.in[k] + i + half);
                const Fr x1 = fr_sub(x1f, x0);
                fr_store(p.out[k] + i, fr_add(x0, fr_mmul(v_mont, x1)));
                // poly *= (x0 + x1 t)
                poly[k + 1] = fr_mmul(poly[k], x1);
#pragma unroll
                for (int d = k; d >= 1; --d) poly[d] = fr_add(fr_mmul(poly[d], x0), fr_mmul(poly[d - 1], x1));
                poly[0] = fr_mmul(poly[0], x0);
            }
#pragma unroll
            for (int d = 0; d <= K; ++d) q[d] = fr_add(q[d], poly[d]);
        }
        if (eq.hi) {
            const Fr eh = fr_load(eq.hi + (base >> eq.kl));
#pragma unroll
            for (int d = 0; d <= K; ++d) q[d] = fr_mmul(q[d], eh);
        }
#pragma unroll
        for (int d = 0; d <= K; ++d) acc[d] = fr_add(acc[d], q[d]);
    }
    // every coefficient is e * (product of K standard values) / R^(K-1)
    grid_sum_finish<K + 1>(acc, partial, ticket, out, (1u << (K + 1)) - 1u, red, K - 1);
}

// ---------------------------------------------------------------------------
// legacy adjacent-pair rounds (proof.cu:12-160).  Pairs (2g, 2g+1); the product
// terms keep the factor 1/R that the reference leaves on them.
// MODE 0: inner product (plain sums)   MODE 1: Hadamard (eq-weighted)   MODE 2: binary
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kThreads) legacy_round_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b,
                                                                 size_t n_in, size_t n_out, Fr v_mont, EqTab eq, unsigned R,
                                                                 Fr* __restrict__ na, Fr* __restrict__ nb,
                                                                 Fr* __restrict__ partial, unsigned* ticket, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc[3];
    acc[0] = acc[1] = acc[2] = fr_zero();
    const size_t lmask = ((size_t)1 << eq.kl) - 1;
    const size_t piece = (size_t)blockDim.x * R;          // never straddles a chunk of the low table
    const size_t npieces = (n_out + piece - 1) / piece;
    for (size_t c = blockIdx.x; c < npieces; c += gridDim.x) {
        Fr q0 = fr_zero(), q1 = fr_zero(), q2 = fr_zero();
        const size_t base = c * piece;
        for (size_t jj = threadIdx.x; jj < piece && base + jj < n_out; jj += blockDim.x) {
            const size_t j = (base + jj) & lmask;
            const size_t g = base + jj;
            const Fr a0 = fr_load(a + 2 * g);
            const Fr a1 = (2 * g + 1 < n_in) ? fr_load(a + 2 * g + 1) : fr_zero();
            const Fr da = fr_sub(a1, a0);
            Fr t0, t1, t2;
            if (MODE == 2) {
                t0 = fr_sub(fr_mmul(a0, a0), a0);
                t1 = fr_sub(fr_mmul(fr_add(a0, a0), da), da);
                t2 = fr_mmul(da, da);
            } else {
                const Fr b0 = fr_load(b + 2 * g);
                const Fr b1 = (2 * g + 1 < n_in) ? fr_load(b + 2 * g + 1) : fr_zero();
                const Fr db = fr_sub(b1, b0);
                t0 = fr_mmul(a0, b0);
                t1 = fr_add(fr_mmul(a0, db), fr_mmul(b0, da));
                t2 = fr_mmul(da, db);
                fr_store(nb + g, fr_add(b0, fr_mmul(v_mont, db)));
            }
            fr_store(na + g, fr_add(a0, fr_mmul(v_mont, da)));
            if (MODE != 0) {
                const Fr e = fr_load(eq.lo + j);
                t0 = fr_mmul(t0, e); t1 = fr_mmul(t1, e); t2 = fr_mmul(t2, e);
            }
            q0 = fr_add(q0, t0); q1 = fr_add(q1, t1); q2 = fr_add(q2, t2);
        }
        if (MODE != 0 && eq.hi) {
            const Fr eh = fr_load(eq.hi + (base >> eq.kl));
            q0 = fr_mmul(q0, eh); q1 = fr_mmul(q1, eh); q2 = fr_mmul(q2, eh);
        }
        acc[0] = fr_add(acc[0], q0); acc[1] = fr_add(acc[1], q1); acc[2] = fr_add(acc[2], q2);
    }
    grid_sum_finish<3>(acc, partial, ticket, out, 0u, red);
}

template <int MODE>
static int legacy_sumcheck(const Fr* d_a, const Fr* d_b, size_t n, const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                           unsigned k, zkb_fr_t* h_proof, cudaStream_t s) {
    if (k > 32) return fail(ZKB_ERR_LIMIT, "sumcheck: more than 32 variables");
    const size_t full = (size_t)1 << k;
    if (n == 0 || n <= full / 2 || n > full) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    Scratch scratch(s);
    const size_t half0 = (n + 1) / 2;
    Fr* buf[2][2];
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 2; ++j) {
            buf[i][j] = scratch.get_n<Fr>(half0);
            if (!buf[i][j]) return ZKB_ERR_CUDA;
        }
    const unsigned max_grid = (unsigned)sm_count() * 4;
    Fr* partial = scratch.get_n<Fr>((size_t)max_grid * 3);
    unsigned* ticket = scratch.get_n<unsigned>(4);
    const size_t n_out_vals = 3 * (size_t)k + 2;
    Fr* d_proof = scratch.get_n<Fr>(n_out_vals);
    if (!partial || !ticket || !d_proof) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
    const Fr* ca = d_a;
    const Fr* cb = d_b;
    size_t n_in = n;
    EqTab tabs[33];
    if (MODE != 0 && k) {
        // the reference requires the half-size arrays to fit their challenges exactly: check before any launch
        size_t ni = n;
        for (unsigned r = 0; r < k; ++r) {
            const size_t no = (ni + 1) / 2, f = (size_t)1 << (k - 1 - r);
            if (no <= f / 2 || no > f) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
            ni = no;
        }
        ZKB_TRY(make_eq_series(h_u + 1, k - 1, k, 1, tabs, scratch, s));
    }
    for (unsigned r = 0; r < k; ++r) {
        const size_t n_out = (n_in + 1) / 2;
        EqTab eq = {nullptr, nullptr, 0};
        if (MODE != 0) {
            // u_ = u[r+1 .. k): k-1-r variables; the reference requires the
            // half-size arrays to fit them exactly
            const unsigned kk = k - 1 - r;
            const size_t f = (size_t)1 << kk;
            if (n_out <= f / 2 || n_out > f) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
            eq = tabs[r];
        } else {
            eq.kl = kEqLoBits;
        }
        const Fr v = dev_fr_mont(MODE == 0 ? h_u[r] : h_v[r]);
        unsigned R, grid;
        pieces_for(n_out, &R, &grid);
        ZKB_LAUNCH(legacy_round_kernel<MODE>, grid, kThreads, 0, s,
                   ca, cb, n_in, n_out, v, eq, R, buf[r & 1][0], buf[r & 1][1], partial, ticket, d_proof + 3 * r);
        ca = buf[r & 1][0];
        cb = buf[r & 1][1];
        n_in = n_out;
    }
    // trailing a(0) [, b(0)]
    ZKB_CUDA(cudaMemcpyAsync(d_proof + 3 * k, ca, 32, cudaMemcpyDeviceToDevice, s));
    if (MODE != 2) ZKB_CUDA(cudaMemcpyAsync(d_proof + 3 * k + 1, cb, 32, cudaMemcpyDeviceToDevice, s));
    ZKB_CUDA(cudaMemcpyAsync(h_proof, d_proof, 32 * (MODE == 2 ? 3 * (size_t)k + 1 : n_out_vals), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

}  // namespace zkb

using namespace zkb;
#define FR(p) reinterpret_cast<Fr*>(p)
#define CFR(p) reinterpret_cast<const Fr*>(p)

extern "C" {

int zkb_zkip(const zkb_fr_t* h_claim, const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n,
             const zkb_fr_t* h_u, unsigned k, zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (k == 0) { *h_final = *h_claim; return ZKB_OK; }
    if (n == 0) return fail(ZKB_ERR_DIM, "zkip: empty input");
    Scratch scratch(s);
    Fr* d_polys = scratch.get_n<Fr>(3 * (size_t)k);
    if (!d_polys) return ZKB_ERR_CUDA;
    ZKB_TRY(zkip_device(CFR(d_a), CFR(d_b), n, h_u, k, k, d_polys, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_polys, d_polys, 96 * (size_t)k, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return zkip_verify(h_claim, h_u, k, h_polys, h_final);
}

int zkb_zkip_stacked(const zkb_fr_t* h_claim, const zkb_fr_t* d_A, const zkb_fr_t* d_B, size_t num, size_t D,
                     const zkb_fr_t* h_uN, const zkb_fr_t* h_vN, unsigned kN, const zkb_fr_t* h_uD, unsigned kD,
                     zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (num == 0 || D == 0) return fail(ZKB_ERR_DIM, "a.size != N * D");
    if (kN > 31) return fail(ZKB_ERR_LIMIT, "zkip_stacked: more than 31 variables over the stack");
    if (kN != clog2(num)) return fail(ZKB_ERR_DIM, "zkip_stacked: uN.size() != ceilLog2(N)");
    if (kN + kD == 0) { *h_final = *h_claim; return ZKB_OK; }
    Scratch scratch(s);
    Fr* d_polys = scratch.get_n<Fr>(3 * ((size_t)kN + kD) + 1);
    if (!d_polys) return ZKB_ERR_CUDA;
    const Fr* ca = CFR(d_A);
    const Fr* cb = CFR(d_B);
    size_t heads = num;
    if (kN) {
        const size_t half0 = (((size_t)1 << kN) >> 1) * D;
        Fr* buf[2][2];
        for (int i = 0; i < 2; ++i)
            for (int j = 0; j < 2; ++j) {
                buf[i][j] = scratch.get_n<Fr>(half0 >> i ? half0 >> i : 1);
                if (!buf[i][j]) return ZKB_ERR_CUDA;
            }
        const unsigned max_grid = grid_for(half0, kThreads, 4);
        Fr* partial = scratch.get_n<Fr>((size_t)max_grid * 3);
        unsigned* ticket = scratch.get_n<unsigned>(4);
        if (!partial || !ticket) return ZKB_ERR_CUDA;
        ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
        // round r weights by eq over uN[0 .. kN - 1 - r), pairs with uN[kN - 1 - r], folds with vN[kN - 1 - r]
        EqTab tabs[33];
        ZKB_TRY(make_eq_series(h_uN, kN - 1, kN, 0, tabs, scratch, s));
        for (unsigned r = 0; r < kN; ++r) {
            const size_t half_heads = ((size_t)1 << (kN - r)) >> 1;
            const size_t half = half_heads * D;
            const Fr v = dev_fr_mont(h_vN[kN - 1 - r]);
            ZKB_LAUNCH(zkip_stacked_round_kernel, grid_for(half, kThreads, 4), kThreads, 0, s, ca, cb, heads * D, half, D, v, tabs[r],
                       buf[r & 1][0], buf[r & 1][1], partial, ticket, d_polys + 3 * r);
            ca = buf[r & 1][0];
            cb = buf[r & 1][1];
            heads = half_heads;
        }
    }
    // what is left is one head: the plain inner-product sumcheck over D
    if (kD) ZKB_TRY(zkip_device(ca, cb, D, h_uD, kD, kD, d_polys + 3 * kN, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_polys, d_polys, 96 * ((size_t)kN + kD), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    // the reference's checks (zkfc.cu:213-219): q = eq(u) * p, claim == q(0) + q(1)
    hfr::H claim = hfr::load(*h_claim);
    for (unsigned r = 0; r < kN; ++r) {
        const hfr::H c[3] = {hfr::load(h_polys[3 * r]), hfr::load(h_polys[3 * r + 1]), hfr::load(h_polys[3 * r + 2])};
        const hfr::H u = hfr::load(h_uN[kN - 1 - r]);
        const hfr::H p1 = hfr::add(hfr::add(c[0], c[1]), c[2]);
        const hfr::H lhs = hfr::add(hfr::mul(hfr::sub(hfr::from_u64(1), u), c[0]), hfr::mul(u, p1));
        if (!hfr::eq(claim, lhs)) return fail(ZKB_ERR_VERIFY, "claim != q(0) + q(1)");
        claim = hfr::poly_eval(c, 3, hfr::load(h_vN[kN - 1 - r]));
    }
    const zkb_fr_t mid = hfr::store(claim);
    if (kD == 0) { *h_final = mid; return ZKB_OK; }
    return zkip_verify(&mid, h_uD, kD, h_polys + 3 * kN, h_final);
}

int zkb_zkip_partial(const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n, const zkb_fr_t* h_u, unsigned k, unsigned rounds,
                     zkb_fr_t* h_sums, zkb_fr_t* h_tail_a, zkb_fr_t* h_tail_b, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (n == 0) return fail(ZKB_ERR_DIM, "zkip: empty input");
    if (rounds > k) return fail(ZKB_ERR_ARG, "zkip: more rounds than challenges");
    const unsigned kn = clog2(n);
    if (rounds > kn) return fail(ZKB_ERR_DIM, "zkip: more rounds than variables");
    Scratch scratch(s);
    Fr* d_polys = scratch.get_n<Fr>(3 * (size_t)rounds + 1);
    if (!d_polys) return ZKB_ERR_CUDA;
    const Fr *fa = nullptr, *fb = nullptr;
    // the challenge of local round r is h_u[k - 1 - r]: present the k - rounds unused ones as absent variables
    ZKB_TRY(zkip_device(CFR(d_a), CFR(d_b), n, h_u + (k - rounds), rounds, rounds, d_polys, scratch, s, &fa, &fb));
    const size_t tail = rounds ? ((size_t)1 << kn) >> rounds : n;
    if (rounds) ZKB_CUDA(cudaMemcpyAsync(h_sums, d_polys, 96 * (size_t)rounds, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaMemcpyAsync(h_tail_a, fa, 32 * tail, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaMemcpyAsync(h_tail_b, fb, 32 * tail, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_zkfc_prove(const zkb_fr_t* d_X, const zkb_fr_t* d_W, const zkb_fr_t* d_Y,
                   size_t B, size_t I, size_t O,
                   const zkb_fr_t* h_u_batch, const zkb_fr_t* h_u_input, const zkb_fr_t* h_u_output,
                   zkb_fr_t* h_polys, zkb_fr_t* h_claims, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (!B || !I || !O) return fail(ZKB_ERR_DIM, "zkFC::prove: empty dimension");
    const unsigned kB = clog2(B), kI = clog2(I), kO = clog2(O);
    // The pass over W (every weight once) runs on the caller's stream; the passes over X and Y and
    // the eq tables, which are much smaller, run beside it on the second stream and join before the
    // rounds.  What the second stream touches is allocated on that stream.
    SideStream* side = side_stream();
    if (!side) return ZKB_ERR_CUDA;
    std::lock_guard<std::mutex> turn(side->busy);
    Scratch scratch(s);
    Scratch side_mem(side->st);
    Drain drain{side->st};   // destroyed first: nothing of the second stream outlives the buffers
    // results gathered on the device: [claim, claim_X, claim_W, polys...]
    Fr* d_res = scratch.get_n<Fr>(3 + 3 * (size_t)kI);
    Fr* w_red = scratch.get_n<Fr>(I);
    unsigned* ticket = scratch.get_n<unsigned>(4);
    Fr* partial = scratch.get_n<Fr>((size_t)sm_count() * 4);
    Fr* y_rows = side_mem.get_n<Fr>(B);
    Fr* x_red = side_mem.get_n<Fr>(I);
    Fr* E_b = side_mem.get_n<Fr>((size_t)1 << kB);
    Fr* E_in = side_mem.get_n<Fr>((size_t)1 << kI);
    Fr* d_claim = side_mem.get_n<Fr>(1);
    unsigned* side_ticket = side_mem.get_n<unsigned>(4);
    Fr* side_partial = side_mem.get_n<Fr>((size_t)sm_count() * 4);
    if (!d_res || !w_red || !ticket || !partial || !y_rows || !x_red || !E_b || !E_in || !d_claim || !side_ticket || !side_partial)
        return ZKB_ERR_CUDA;
    // the caller's inputs are ready at this point of the caller's stream
    ZKB_CUDA(cudaEventRecord(side->fork, s));
    ZKB_CUDA(cudaStreamWaitEvent(side->st, side->fork, 0));
    {
        cudaStream_t t = side->st;
        ZKB_TRY(build_eq_table(h_u_batch, kB, E_b, t));
        ZKB_TRY(build_eq_table(h_u_input, kI, E_in, t));
        // claim = Y(u_batch, u_output): row dots with eq(u_output), then eq(u_batch)
        if (kO) ZKB_TRY(partial_me_device(CFR(d_Y), B * O, B, O, 1, h_u_output, kO, y_rows, side_mem, t));
        else ZKB_CUDA(cudaMemcpyAsync(y_rows, d_Y, B * 32, cudaMemcpyDeviceToDevice, t));
        ZKB_CUDA(cudaMemsetAsync(side_ticket, 0, 16, t));
        ZKB_LAUNCH(fr_dot_kernel, grid_for(B, kThreads, 4), kThreads, 0, t, y_rows, E_b, B, side_partial, side_ticket, d_claim, 0u);
        // X_red = eq(u_batch)^T X
        if (kB) ZKB_TRY(partial_me_device(CFR(d_X), B * I, 1, B, I, h_u_batch, kB, x_red, side_mem, t));
        else ZKB_CUDA(cudaMemcpyAsync(x_red, d_X, I * 32, cudaMemcpyDeviceToDevice, t));
        ZKB_CUDA(cudaEventRecord(side->join, t));
    }
    // W_red = W eq(u_output)
    ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
    if (kO) ZKB_TRY(partial_me_device(CFR(d_W), I * O, I, O, 1, h_u_output, kO, w_red, scratch, s));
    else ZKB_CUDA(cudaMemcpyAsync(w_red, d_W, I * 32, cudaMemcpyDeviceToDevice, s));
    ZKB_CUDA(cudaStreamWaitEvent(s, side->join, 0));
    ZKB_CUDA(cudaMemcpyAsync(d_res, d_claim, 32, cudaMemcpyDeviceToDevice, s));
    ZKB_TRY(zkip_device(x_red, w_red, I, h_u_input, kI, kI, d_res + 3, scratch, s));
    ZKB_LAUNCH(fr_dot_kernel, grid_for(I, kThreads, 4), kThreads, 0, s, x_red, E_in, I, partial, ticket, d_res + 1, 0u);
    ZKB_LAUNCH(fr_dot_kernel, grid_for(I, kThreads, 4), kThreads, 0, s, w_red, E_in, I, partial, ticket, d_res + 2, 0u);
    std::vector<zkb_fr_t> res(3 + 3 * (size_t)kI);
    ZKB_CUDA(cudaMemcpyAsync(res.data(), d_res, res.size() * 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    for (size_t i = 0; i < 3 * (size_t)kI; ++i) h_polys[i] = res[3 + i];
    h_claims[0] = res[0];
    h_claims[2] = res[1];
    h_claims[3] = res[2];
    ZKB_TRY(zkip_verify(&res[0], h_u_input, kI, h_polys, &h_claims[1]));
    const hfr::H prod = hfr::mul(hfr::load(res[1]), hfr::load(res[2]));
    if (!hfr::eq(prod, hfr::load(h_claims[1]))) return fail(ZKB_ERR_VERIFY, "Claim does not match");
    return ZKB_OK;
}

int zkb_tlookup_prep(const uint32_t* d_indices, size_t D, size_t N, zkb_fr_t* d_m, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (!N) return ZKB_OK;
    Scratch scratch(s);
    uint32_t* counts = scratch.get_n<uint32_t>(N);
    if (!counts) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemsetAsync(counts, 0, N * 4, s));
    if (D) ZKB_LAUNCH(tl_count_kernel, grid_for(D, kThreads), kThreads, 0, s, d_indices, D, N, counts);
    ZKB_LAUNCH(tl_counts_to_fr_kernel, grid_for(N, kThreads), kThreads, 0, s, counts, N, FR(d_m));
    return ZKB_OK;
}
int zkb_tlookup_range_indices(const zkb_fr_t* d_vals, int32_t low, uint32_t* d_indices, size_t D, void* stream) {
    if (!D) return ZKB_OK;
    hfr::H l = low >= 0 ? hfr::from_u64((uint64_t)low) : hfr::neg(hfr::from_u64((uint64_t)(-(int64_t)low)));
    ZKB_LAUNCH(tl_range_indices_kernel, grid_for(D, kThreads), kThreads, 0, as_stream(stream), CFR(d_vals), dev_fr(l), d_indices, D);
    return ZKB_OK;
}
int zkb_tlookup_range_table(int32_t low, size_t len, size_t table_size, zkb_fr_t* d_table, void* stream) {
    if (!table_size) return ZKB_OK;
    ZKB_LAUNCH(tl_range_table_kernel, grid_for(table_size, kThreads), kThreads, 0, as_stream(stream), (int)low, len, table_size, FR(d_table));
    return ZKB_OK;
}

}  // extern "C"

// Queues the first `run` rounds of the lookup sumcheck (tlookup.cu:281-322) on `s`:
// the inverses A = 1/(S + beta), B = 1/(T + beta), the sum of B * m into d_sums[0] and
// 11 sums per round into d_sums[1 + 11 r].  fin[0..4] receive device pointers to
// A, S, B, T, m as folded by the last round queued.
// d_idx (optional): for every S[i] the table index the caller says holds it; with it the first
// phase-1 round forms A from the N inverses of the table (tl_phase1_first_kernel).
static int tlookup_rounds_device(const Fr* d_S, const Fr* d_table, const Fr* d_m, size_t D, size_t N, const zkb_fr_t* h_beta,
                                 const zkb_fr_t* h_u, const zkb_fr_t* h_v, unsigned run, Fr* d_sums, const Fr* fin[5],
                                 Scratch& scratch, cudaStream_t s, const uint32_t* d_idx = nullptr) {
    const unsigned kD = clog2(D), kN = clog2(N), k1 = kD - kN;
    const bool fused_first = d_idx != nullptr && k1 >= 1 && run >= 1;
    // working arrays: A (D) unless the first round forms it, then ping-pong halves
    Fr* A = fused_first ? nullptr : scratch.get_n<Fr>(D);
    Fr* Bv = scratch.get_n<Fr>(N);
    if ((!fused_first && !A) || !Bv) return ZKB_ERR_CUDA;
    if (!fused_first) ZKB_TRY(zkb_fr_inv_shifted(reinterpret_cast<const zkb_fr_t*>(d_S), h_beta, reinterpret_cast<zkb_fr_t*>(A), D, s));
    ZKB_TRY(zkb_fr_inv_shifted(reinterpret_cast<const zkb_fr_t*>(d_table), h_beta, reinterpret_cast<zkb_fr_t*>(Bv), N, s));
    const size_t half0 = D > 1 ? D / 2 : 1;
    Fr* pp[2][5];
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 5; ++j) {
            // A,S halves shrink from D/2; B,T,m from N/2
            const size_t sz = j < 2 ? (half0 >> i ? half0 >> i : 1) : ((N / 2) >> i ? (N / 2) >> i : 1);
            pp[i][j] = scratch.get_n<Fr>(sz);
            if (!pp[i][j]) return ZKB_ERR_CUDA;
        }
    const unsigned max_grid = (unsigned)sm_count() * 4;
    Fr* partial = scratch.get_n<Fr>((size_t)max_grid * 11);
    unsigned* ticket = scratch.get_n<unsigned>(4);
    if (!partial || !ticket) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
    // sum B*m
    ZKB_LAUNCH(fr_dot_kernel, grid_for(N, kThreads, 4), kThreads, 0, s, Bv, d_m, N, partial, ticket, d_sums, 1u);
    const Fr beta = dev_fr(hfr::load(*h_beta));
    const Fr* cA = A;
    const Fr* cS = d_S;
    const Fr* cB = Bv;
    const Fr* cT = d_table;
    const Fr* cm = d_m;
    size_t M = D;
    EqTab tabs[33];
    if (kD) ZKB_TRY(make_eq_series(h_u, kD - 1, kD, 0, tabs, scratch, s));
    for (unsigned r = 0; r < run; ++r) {
        const size_t half = M / 2;
        const EqTab eq = tabs[r];
        unsigned R, grid;
        pieces_for(half, &R, &grid);
        Fr* out = d_sums + 1 + 11 * (size_t)r;
        const int pb = r & 1;
        if (r < k1) {
            const Fr v = dev_fr_mont(h_v[k1 - 1 - r]);
            if (r == 0 && fused_first) {
                ZKB_LAUNCH(tl_phase1_first_kernel, grid, kThreads, 0, s, cS, d_idx, d_table, Bv, N, half, beta, v, eq, R,
                           pp[pb][0], pp[pb][1], partial, ticket, out);
            } else {
                ZKB_LAUNCH(tl_phase1_kernel, grid, kThreads, 0, s, cA, cS, half, beta, v, eq, R,
                           pp[pb][0], pp[pb][1], partial, ticket, out);
            }
            cA = pp[pb][0]; cS = pp[pb][1];
        } else if (half <= kTlTailHalf && kD - r <= kTlTailRounds) {
            // the remaining phase-2 rounds in one launch
            TlTail tt;
            memset(&tt, 0, sizeof(tt));
            const Fr* cur[5] = {cA, cS, cB, cT, cm};
            const unsigned rounds = run - r;
            for (int a = 0; a < 5; ++a) {
                tt.cur[a] = cur[a];
                for (int par = 0; par < 2; ++par) {
                    tt.nxt[par][a] = scratch.get_n<Fr>(half);
                    if (!tt.nxt[par][a]) return ZKB_ERR_CUDA;
                }
            }
            for (unsigned t = 0; t < rounds; ++t) {
                tt.lo[t] = tabs[r + t].lo;
                tt.v[t] = dev_fr_mont(h_v[kD - 1 - (r + t - k1)]);
            }
            ZKB_LAUNCH(tl_phase2_tail_kernel, 1, 128, 0, s, tt, half, beta, rounds, out);
            const int last = (rounds - 1) & 1;
            cA = tt.nxt[last][0]; cS = tt.nxt[last][1]; cB = tt.nxt[last][2]; cT = tt.nxt[last][3]; cm = tt.nxt[last][4];
            break;
        } else {
            const Fr v = dev_fr_mont(h_v[kD - 1 - (r - k1)]);
            const int qb = (r - k1) & 1;   // B, T, m start shrinking at the first phase-2 round
            ZKB_LAUNCH(tl_phase2_kernel, grid, kThreads, 0, s, cA, cS, cB, cT, cm, half, beta, v, eq, R,
                       pp[pb][0], pp[pb][1], pp[qb][2], pp[qb][3], pp[qb][4], partial, ticket, out);
            cA = pp[pb][0]; cS = pp[pb][1]; cB = pp[qb][2]; cT = pp[qb][3]; cm = pp[qb][4];
        }
        M = half;
    }
    fin[0] = cA; fin[1] = cS; fin[2] = cB; fin[3] = cT; fin[4] = cm;
    return ZKB_OK;
}

// All log2(N) rounds of multi_hadamard_sumchecks (proof.cu:190-241) on the device: round r pairs entry g with g + M/2,
// weights the K + 1 coefficients of prod_k (X_k[g] + t (X_k[g + M/2] - X_k[g])) by eq over the variables below the
// current one (u[0 .. kN-1-r)) and folds with v[kN-1-r].  d_sums receives K + 1 sums per round; fin[j] points at the one
// entry of tensor j that is left (the input itself when N is 1).
static int hadamard_rounds_device(const zkb_fr_t* const* h_d_Xs, unsigned K, size_t N, const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                                  Fr* d_sums, const Fr** fin, Scratch& scratch, cudaStream_t s) {
    const unsigned kN = clog2(N);
    HadamardPtrs ptrs;
    for (unsigned j = 0; j < K; ++j) ptrs.in[j] = CFR(h_d_Xs[j]);
    if (kN) {
        Fr* bufs[2][kMaxHadamard];
        for (int i = 0; i < 2; ++i)
            for (unsigned j = 0; j < K; ++j) {
                bufs[i][j] = scratch.get_n<Fr>((N / 2) >> i ? (N / 2) >> i : 1);
                if (!bufs[i][j]) return ZKB_ERR_CUDA;
            }
        const unsigned max_grid = (unsigned)sm_count() * 4;
        Fr* partial = scratch.get_n<Fr>((size_t)max_grid * (K + 1));
        unsigned* ticket = scratch.get_n<unsigned>(4);
        if (!partial || !ticket) return ZKB_ERR_CUDA;
        ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
        size_t M = N;
        EqTab tabs[33];
        ZKB_TRY(make_eq_series(h_u, kN - 1, kN, 0, tabs, scratch, s));
        for (unsigned r = 0; r < kN; ++r) {
            const size_t half = M / 2;
            const EqTab eq = tabs[r];
            for (unsigned j = 0; j < K; ++j) ptrs.out[j] = bufs[r & 1][j];
            const Fr v = dev_fr_mont(h_v[kN - 1 - r]);
            unsigned R, grid;
            pieces_for(half, &R, &grid);
            Fr* out = d_sums + (size_t)r * (K + 1);
            switch (K) {
                case 1: ZKB_LAUNCH(hadamard_round_kernel<1>, grid, kThreads, 0, s, ptrs, half, v, eq, R, partial, ticket, out); break;
                case 2: ZKB_LAUNCH(hadamard_round_kernel<2>, grid, kThreads, 0, s, ptrs, half, v, eq, R, partial, ticket, out); break;
                case 3: ZKB_LAUNCH(hadamard_round_kernel<3>, grid, kThreads, 0, s, ptrs, half, v, eq, R, partial, ticket, out); break;
                case 4: ZKB_LAUNCH(hadamard_round_kernel<4>, grid, kThreads, 0, s, ptrs, half, v, eq, R, partial, ticket, out); break;
                case 5: ZKB_LAUNCH(hadamard_round_kernel<5>, grid, kThreads, 0, s, ptrs, half, v, eq, R, partial, ticket, out); break;
                default: ZKB_LAUNCH(hadamard_round_kernel<6>, grid, kThreads, 0, s, ptrs, half, v, eq, R, partial, ticket, out); break;
            }
            for (unsigned j = 0; j < K; ++j) ptrs.in[j] = bufs[r & 1][j];
            M = half;
        }
    }
    for (unsigned j = 0; j < K; ++j) fin[j] = ptrs.in[j];
    return ZKB_OK;
}

extern "C" {

int zkb_tlookup_partial(const zkb_fr_t* d_S, const zkb_fr_t* d_table, const zkb_fr_t* d_m, size_t D, size_t N,
                        const zkb_fr_t* h_beta, const zkb_fr_t* h_u, const zkb_fr_t* h_v, unsigned rounds,
                        zkb_fr_t* h_sums, zkb_fr_t* h_tails, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (!D || !N || (D & (D - 1)) || (N & (N - 1)) || D % N)
        return fail(ZKB_ERR_DIM, "D or N is not power of 2, or D is not divisible by N");
    const unsigned kD = clog2(D), kN = clog2(N), k1 = kD - kN;
    if (kD > 32) return fail(ZKB_ERR_LIMIT, "tLookup: D above 2^32");
    if (rounds > kD) return fail(ZKB_ERR_ARG, "tLookup: more rounds than variables");
    Scratch scratch(s);
    Fr* d_sums = scratch.get_n<Fr>(1 + 11 * (size_t)rounds);
    if (!d_sums) return ZKB_ERR_CUDA;
    const Fr* fin[5];
    ZKB_TRY(tlookup_rounds_device(CFR(d_S), CFR(d_table), CFR(d_m), D, N, h_beta, h_u, h_v, rounds, d_sums, fin, scratch, s));
    const size_t nAS = D >> rounds, nBT = rounds > k1 ? N >> (rounds - k1) : N;
    ZKB_CUDA(cudaMemcpyAsync(h_sums, d_sums, (1 + 11 * (size_t)rounds) * 32, cudaMemcpyDeviceToHost, s));
    size_t off = 0;
    for (int a = 0; a < 5; ++a) {
        const size_t cnt = a < 2 ? nAS : nBT;
        ZKB_CUDA(cudaMemcpyAsync(h_tails + off, fin[a], cnt * 32, cudaMemcpyDeviceToHost, s));
        off += cnt;
    }
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_tlookup_prove(const zkb_fr_t* d_S, const zkb_fr_t* d_table, const zkb_fr_t* d_m,
                      size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_beta,
                      const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                      zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    return zkb_tlookup_prove_indexed(d_S, nullptr, d_table, d_m, D, N, h_alpha, h_beta, h_u, h_v, h_polys, h_final, stream);
}

int zkb_tlookup_prove_indexed(const zkb_fr_t* d_S, const uint32_t* d_indices, const zkb_fr_t* d_table, const zkb_fr_t* d_m,
                              size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_beta,
                              const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                              zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (!D || !N || (D & (D - 1)) || (N & (N - 1)) || D % N)
        return fail(ZKB_ERR_DIM, "D or N is not power of 2, or D is not divisible by N");
    const unsigned kD = clog2(D), kN = clog2(N), k1 = kD - kN;
    if (kD > 32) return fail(ZKB_ERR_LIMIT, "tLookup: D above 2^32");
    Scratch scratch(s);
    Fr* d_sums = scratch.get_n<Fr>(1 + 11 * (size_t)kD);
    if (!d_sums) return ZKB_ERR_CUDA;
    const Fr* fin[5];
    ZKB_TRY(tlookup_rounds_device(CFR(d_S), CFR(d_table), CFR(d_m), D, N, h_beta, h_u, h_v, kD, d_sums, fin, scratch, s, d_indices));
    std::vector<zkb_fr_t> sums(1 + 11 * (size_t)kD);
    ZKB_CUDA(cudaMemcpyAsync(sums.data(), d_sums, sums.size() * 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));

    // host: assemble the round polynomials and replay the checks
    return tlookup_assemble(sums.data(), D, N, h_alpha, h_u, h_v, h_polys, h_final);
}

int zkb_multi_hadamard(const zkb_fr_t* h_claim, const zkb_fr_t* const* h_d_Xs, unsigned K, size_t N,
                       const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                       zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (K < 1 || K > (unsigned)kMaxHadamard) return fail(ZKB_ERR_LIMIT, "multi_hadamard: between 1 and 6 tensors");
    if (N == 1) { *h_final = *h_claim; return ZKB_OK; }
    if (N == 0 || (N & (N - 1))) return fail(ZKB_ERR_DIM, "N is not a power of 2");
    const unsigned kN = clog2(N);
    Scratch scratch(s);
    Fr* d_sums = scratch.get_n<Fr>((size_t)kN * (K + 1));
    if (!d_sums) return ZKB_ERR_CUDA;
    const Fr* fin[kMaxHadamard];
    ZKB_TRY(hadamard_rounds_device(h_d_Xs, K, N, h_u, h_v, d_sums, fin, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_polys, d_sums, (size_t)kN * (K + 1) * 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return hadamard_replay(h_claim, h_polys, K, kN, h_u, h_v, h_final);
}

int zkb_multi_hadamard_partial(const zkb_fr_t* const* h_d_Xs, unsigned K, size_t N, const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                               zkb_fr_t* h_sums, zkb_fr_t* h_tails, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (K < 1 || K > (unsigned)kMaxHadamard) return fail(ZKB_ERR_LIMIT, "multi_hadamard: between 1 and 6 tensors");
    if (N == 0 || (N & (N - 1))) return fail(ZKB_ERR_DIM, "N is not a power of 2");
    const unsigned kN = clog2(N);
    Scratch scratch(s);
    Fr* d_sums = scratch.get_n<Fr>((size_t)kN * (K + 1) + 1);
    if (!d_sums) return ZKB_ERR_CUDA;
    const Fr* fin[kMaxHadamard];
    ZKB_TRY(hadamard_rounds_device(h_d_Xs, K, N, h_u, h_v, d_sums, fin, scratch, s));
    if (kN) ZKB_CUDA(cudaMemcpyAsync(h_sums, d_sums, (size_t)kN * (K + 1) * 32, cudaMemcpyDeviceToHost, s));
    for (unsigned j = 0; j < K; ++j) ZKB_CUDA(cudaMemcpyAsync(h_tails + j, fin[j], 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_hadamard_product_sumcheck(const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n,
                                  const zkb_fr_t* h_u, const zkb_fr_t* h_v, unsigned k,
                                  zkb_fr_t* h_proof, void* stream) {
    return legacy_sumcheck<1>(CFR(d_a), CFR(d_b), n, h_u, h_v, k, h_proof, as_stream(stream));
}
int zkb_inner_product_sumcheck(const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n,
                               const zkb_fr_t* h_u, unsigned k, zkb_fr_t* h_proof, void* stream) {
    return legacy_sumcheck<0>(CFR(d_a), CFR(d_b), n, h_u, nullptr, k, h_proof, as_stream(stream));
}
int zkb_binary_sumcheck(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                        unsigned k, zkb_fr_t* h_proof, void* stream) {
    return legacy_sumcheck<2>(CFR(d_a), CFR(d_a), n, h_u, h_v, k, h_proof, as_stream(stream));
}

// ---- provers with the data dealt out over the ranks of the communicator (comm.cu) ----
// eq(u[0..nbits); index): challenge j pairs with bit j of the index
static hfr::H rank_weight(const zkb_fr_t* u, unsigned nbits, size_t index) {
    hfr::H w = hfr::from_u64(1);
    const hfr::H one = hfr::from_u64(1);
    for (unsigned j = 0; j < nbits; ++j) {
        const hfr::H uj = hfr::load(u[j]);
        w = hfr::mul(w, ((index >> j) & 1) ? uj : hfr::sub(one, uj));
    }
    return w;
}

int zkb_zkfc_prove_sharded(const zkb_fr_t* d_X_local, const zkb_fr_t* d_W_local, const zkb_fr_t* d_Y,
                           size_t B, size_t I_local, size_t O,
                           const zkb_fr_t* h_u_batch, const zkb_fr_t* h_u_input, const zkb_fr_t* h_u_output,
                           zkb_fr_t* h_polys, zkb_fr_t* h_claims, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    const int world = comm_world();
    if (world < 1) return fail(ZKB_ERR_ARG, "comm: not initialised (zkb_comm_init)");
    if (world & (world - 1)) return fail(ZKB_ERR_ARG, "zkFC::prove: the number of ranks must be a power of two");
    if (!B || !I_local || !O) return fail(ZKB_ERR_DIM, "zkFC::prove: empty dimension");
    if (I_local & (I_local - 1)) return fail(ZKB_ERR_DIM, "zkFC::prove: a rank's share of the input dimension must be a power of two");
    const unsigned kP = clog2((size_t)world), kL = clog2(I_local), kI = kL + kP, kB = clog2(B), kO = clog2(O);
    const size_t block = 3 * (size_t)kL + 4;            // local round sums, surviving pair, X and W claims of the share
    Scratch scratch(s);
    Fr* d_part = scratch.get_n<Fr>(block + 1);          // + the claim on Y
    Fr* d_all = scratch.get_n<Fr>(block * world);
    Fr* y_rows = scratch.get_n<Fr>(B);
    Fr* x_red = scratch.get_n<Fr>(I_local);
    Fr* w_red = scratch.get_n<Fr>(I_local);
    Fr* E_b = scratch.get_n<Fr>((size_t)1 << kB);
    Fr* E_in = scratch.get_n<Fr>((size_t)1 << kL);
    unsigned* ticket = scratch.get_n<unsigned>(4);
    Fr* partial = scratch.get_n<Fr>((size_t)sm_count() * 4);
    if (!d_part || !d_all || !y_rows || !x_red || !w_red || !E_b || !E_in || !ticket || !partial) return ZKB_ERR_CUDA;
    ZKB_TRY(build_eq_table(h_u_batch, kB, E_b, s));
    ZKB_TRY(build_eq_table(h_u_input + kP, kL, E_in, s));   // the challenges above the rank's own index bits
    if (kO) ZKB_TRY(partial_me_device(CFR(d_Y), B * O, B, O, 1, h_u_output, kO, y_rows, scratch, s));
    else ZKB_CUDA(cudaMemcpyAsync(y_rows, d_Y, B * 32, cudaMemcpyDeviceToDevice, s));
    ZKB_CUDA(cudaMemsetAsync(ticket, 0, 16, s));
    ZKB_LAUNCH(fr_dot_kernel, grid_for(B, kThreads, 4), kThreads, 0, s, y_rows, E_b, B, partial, ticket, d_part + block, 0u);
    if (kB) ZKB_TRY(partial_me_device(CFR(d_X_local), B * I_local, 1, B, I_local, h_u_batch, kB, x_red, scratch, s));
    else ZKB_CUDA(cudaMemcpyAsync(x_red, d_X_local, I_local * 32, cudaMemcpyDeviceToDevice, s));
    if (kO) ZKB_TRY(partial_me_device(CFR(d_W_local), I_local * O, I_local, O, 1, h_u_output, kO, w_red, scratch, s));
    else ZKB_CUDA(cudaMemcpyAsync(w_red, d_W_local, I_local * 32, cudaMemcpyDeviceToDevice, s));
    // local round r uses the challenge h_u_input[kI - 1 - r]
    const Fr *fa = nullptr, *fb = nullptr;
    ZKB_TRY(zkip_device(x_red, w_red, I_local, h_u_input + kP, kL, kL, d_part, scratch, s, &fa, &fb));
    ZKB_CUDA(cudaMemcpyAsync(d_part + 3 * kL, fa, 32, cudaMemcpyDeviceToDevice, s));
    ZKB_CUDA(cudaMemcpyAsync(d_part + 3 * kL + 1, fb, 32, cudaMemcpyDeviceToDevice, s));
    ZKB_LAUNCH(fr_dot_kernel, grid_for(I_local, kThreads, 4), kThreads, 0, s, x_red, E_in, I_local, partial, ticket, d_part + 3 * kL + 2, 0u);
    ZKB_LAUNCH(fr_dot_kernel, grid_for(I_local, kThreads, 4), kThreads, 0, s, w_red, E_in, I_local, partial, ticket, d_part + 3 * kL + 3, 0u);
    ZKB_TRY(comm_allgather(d_part, d_all, block * 32, s));
    std::vector<zkb_fr_t> all(block * world), claim(1);
    ZKB_CUDA(cudaMemcpyAsync(all.data(), d_all, all.size() * 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaMemcpyAsync(claim.data(), d_part + block, 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    // every rank: sums added, the last log2(world) rounds on the surviving pairs, the verifier's checks
    const size_t zk_block = 3 * (size_t)kL + 2;
    std::vector<zkb_fr_t> parts(zk_block * world);
    for (int p = 0; p < world; ++p) memcpy(&parts[p * zk_block], &all[p * block], zk_block * 32);
    ZKB_TRY(zkb_zkip_combine(parts.data(), (unsigned)world, kI, h_u_input, claim.data(), h_polys, &h_claims[1]));
    hfr::H cx = hfr::zero(), cw = hfr::zero();
    for (int p = 0; p < world; ++p) {
        const hfr::H w = rank_weight(h_u_input, kP, (size_t)p);
        cx = hfr::add(cx, hfr::mul(w, hfr::load(all[p * block + zk_block])));
        cw = hfr::add(cw, hfr::mul(w, hfr::load(all[p * block + zk_block + 1])));
    }
    h_claims[0] = claim[0];
    h_claims[2] = hfr::store(cx);
    h_claims[3] = hfr::store(cw);
    if (!hfr::eq(hfr::mul(cx, cw), hfr::load(h_claims[1]))) return fail(ZKB_ERR_VERIFY, "Claim does not match");
    return ZKB_OK;
}

int zkb_tlookup_prove_sharded(const zkb_fr_t* d_S_local, const zkb_fr_t* d_table_local, const zkb_fr_t* d_m_local,
                              size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_beta,
                              const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                              zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    const int world = comm_world();
    if (world < 1) return fail(ZKB_ERR_ARG, "comm: not initialised (zkb_comm_init)");
    if (world & (world - 1)) return fail(ZKB_ERR_ARG, "tLookup: the number of ranks must be a power of two");
    if (!D || !N || (D & (D - 1)) || (N & (N - 1)) || D % N)
        return fail(ZKB_ERR_DIM, "D or N is not power of 2, or D is not divisible by N");
    if (N < (size_t)world) return fail(ZKB_ERR_DIM, "tLookup: more ranks than table entries");
    const unsigned kD = clog2(D), kN = clog2(N), k1 = kD - kN, kP = clog2((size_t)world);
    if (kD > 32) return fail(ZKB_ERR_LIMIT, "tLookup: D above 2^32");
    const unsigned rounds = kD - kP;
    // a rank's challenges: u above its own index bits; v without the entries of the shared last rounds
    std::vector<zkb_fr_t> vl;
    for (unsigned i = 0; i < k1; ++i) vl.push_back(h_v[i]);
    for (unsigned i = k1 + kP; i < kD; ++i) vl.push_back(h_v[i]);
    if (vl.empty()) vl.resize(1);
    const size_t block = 1 + 11 * (size_t)rounds + 5;
    Scratch scratch(s);
    Fr* d_part = scratch.get_n<Fr>(block);
    Fr* d_all = scratch.get_n<Fr>(block * world);
    if (!d_part || !d_all) return ZKB_ERR_CUDA;
    const Fr* fin[5];
    ZKB_TRY(tlookup_rounds_device(CFR(d_S_local), CFR(d_table_local), CFR(d_m_local), D / world, N / world, h_beta,
                                  h_u + kP, vl.data(), rounds, d_part, fin, scratch, s));
    for (int a = 0; a < 5; ++a)
        ZKB_CUDA(cudaMemcpyAsync(d_part + 1 + 11 * (size_t)rounds + a, fin[a], 32, cudaMemcpyDeviceToDevice, s));
    ZKB_TRY(comm_allgather(d_part, d_all, block * 32, s));
    std::vector<zkb_fr_t> all(block * world);
    ZKB_CUDA(cudaMemcpyAsync(all.data(), d_all, all.size() * 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return zkb_tlookup_combine(all.data(), (unsigned)world, D, N, h_alpha, h_beta, h_u, h_v, h_polys, h_final);
}

int zkb_multi_hadamard_sharded(const zkb_fr_t* h_claim, const zkb_fr_t* const* h_d_Xs_local, unsigned K, size_t N,
                               const zkb_fr_t* h_u, const zkb_fr_t* h_v, zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    const int world = comm_world();
    if (world < 1) return fail(ZKB_ERR_ARG, "comm: not initialised (zkb_comm_init)");
    if (world & (world - 1)) return fail(ZKB_ERR_ARG, "multi_hadamard: the number of ranks must be a power of two");
    if (K < 1 || K > (unsigned)kMaxHadamard) return fail(ZKB_ERR_LIMIT, "multi_hadamard: between 1 and 6 tensors");
    if (N == 0 || (N & (N - 1))) return fail(ZKB_ERR_DIM, "N is not a power of 2");
    if (N < (size_t)world) return fail(ZKB_ERR_DIM, "multi_hadamard: more ranks than entries");
    const unsigned kN = clog2(N), kP = clog2((size_t)world), local = kN - kP;
    const size_t block = (size_t)local * (K + 1) + K;     // this rank's sums, then its K surviving entries
    Scratch scratch(s);
    Fr* d_part = scratch.get_n<Fr>(block);
    Fr* d_all = scratch.get_n<Fr>(block * world);
    if (!d_part || !d_all) return ZKB_ERR_CUDA;
    const Fr* fin[kMaxHadamard];
    // a rank's own rounds bind the variables above its index bits
    ZKB_TRY(hadamard_rounds_device(h_d_Xs_local, K, N / world, h_u + kP, h_v + kP, d_part, fin, scratch, s));
    for (unsigned j = 0; j < K; ++j)
        ZKB_CUDA(cudaMemcpyAsync(d_part + (size_t)local * (K + 1) + j, fin[j], 32, cudaMemcpyDeviceToDevice, s));
    ZKB_TRY(comm_allgather(d_part, d_all, block * 32, s));
    std::vector<zkb_fr_t> all(block * world);
    ZKB_CUDA(cudaMemcpyAsync(all.data(), d_all, all.size() * 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return zkb_multi_hadamard_combine(all.data(), (unsigned)world, K, kN, h_u, h_v, h_claim, h_polys, h_final);
}

}  // extern "C"
