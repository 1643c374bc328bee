// Device helpers shared by the Fr kernels: warp/block reductions, equality
// ("eq") tables for multilinear extensions, grid sizing.
#pragma once
#include "common.cuh"
#include "field.cuh"

namespace zkb {

using FrP = FrParams;

ZKB_DEV Fr fr_add(const Fr& a, const Fr& b) { return fe_add<FrP>(a, b); }
ZKB_DEV Fr fr_sub(const Fr& a, const Fr& b) { return fe_sub<FrP>(a, b); }
ZKB_DEV Fr fr_neg(const Fr& a) { return fe_neg<FrP>(a); }
ZKB_DEV Fr fr_mmul(const Fr& a, const Fr& b) { return mont_mul<FrP>(a, b); }   // a*b*R^-1
ZKB_DEV Fr fr_zero() { return fe_zero<FrP>(); }
ZKB_DEV Fr fr_load(const Fr* p) { return fe_load<FrP>(p); }
ZKB_DEV void fr_store(Fr* p, const Fr& a) { fe_store<FrP>(p, a); }

// a + x*(b - a) with x in Montgomery form: one multilinear fold of a pair
ZKB_DEV Fr fr_fold(const Fr& a, const Fr& b, const Fr& x_mont) {
    return fr_add(a, fr_mmul(x_mont, fr_sub(b, a)));
}

ZKB_DEV Fr fr_shfl_down(const Fr& v, int off) {
    Fr o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = __shfl_down_sync(0xffffffffu, v.v[i], off);
    return o;
}
ZKB_DEV Fr warp_sum(Fr v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fr_add(v, fr_shfl_down(v, off));
    return v;   // lane 0 holds the sum
}
// Sum over the block; `smem` has room for 32 Fr.  Valid in thread 0.
// Ends with a barrier so that `smem` can be reused at once.
ZKB_DEV Fr block_sum(Fr v, Fr* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    Fr r = fr_zero();
    if (warp == 0) {
        if (lane < nwarps) r = smem[lane];
        r = warp_sum(r);
    }
    __syncthreads();
    return r;
}

// Sum of x_j * E_j where E_j is a Montgomery-form weight and most x_j are small
// signed integers held as field elements (fixed-point tensors: |x| < 2^64, a
// negative value stored as r - |x|).  A small x costs two carry chains of 8
// 32x32 multiply-adds (four chains above 2^32) into an unreduced 352-bit
// accumulator instead of a 256-multiply-add Montgomery product; a negative x
// is accumulated as |x| * (r - E), the same residue.  Anything that is not small
// goes through the field product.  finish() returns sum x_j * e_j (e = E / R) as a
// field element.  Room: a term is below 2^320, so 2^32 terms fit.
struct LazyDot {
    uint32_t acc[11];
    Fr gen;
    ZKB_DEV void init() {
#pragma unroll
        for (int i = 0; i < 11; ++i) acc[i] = 0u;
        gen = fr_zero();
    }
    // acc += x * e * 2^(32 * SH)
    template <int SH>
    ZKB_DEV void mac(uint32_t x, const Fr& e) {
        ptx_mad_lo_cc(acc[SH], e.v[0], x);
#pragma unroll
        for (int i = 1; i < 8; ++i) ptx_madc_lo_cc(acc[SH + i], e.v[i], x);
#pragma unroll
        for (int i = SH + 8; i < 10; ++i) ptx_addc_cc(acc[i], 0u);
        ptx_addc(acc[10], 0u);
        ptx_mad_hi_cc(acc[SH + 1], e.v[0], x);
#pragma unroll
        for (int i = 1; i < 8; ++i) ptx_madc_hi_cc(acc[SH + 1 + i], e.v[i], x);
#pragma unroll
        for (int i = SH + 9; i < 10; ++i) ptx_addc_cc(acc[i], 0u);
        if (SH + 9 <= 10) ptx_addc(acc[10], 0u);
    }
    // r - a as plain integers (a in [0, r])
    ZKB_DEV static Fr rsub(const Fr& a) {
        Fr d;
        d.v[0] = ptx_sub_cc3(FrP::mod(0), a.v[0]);
#pragma unroll
        for (int i = 1; i < 7; ++i) d.v[i] = ptx_subc_cc3(FrP::mod(i), a.v[i]);
        d.v[7] = ptx_subc3(FrP::mod(7), a.v[7]);
        return d;
    }
    ZKB_DEV void add(const Fr& x, const Fr& e) {
        uint32_t m0 = x.v[0], m1 = x.v[1];
        Fr w = e;
        bool small = (x.v[2] | x.v[3] | x.v[4] | x.v[5] | x.v[6] | x.v[7]) == 0u;
        if (!small) {
            const Fr m = rsub(x);
            if ((m.v[2] | m.v[3] | m.v[4] | m.v[5] | m.v[6] | m.v[7]) == 0u) {
                small = true;
                m0 = m.v[0]; m1 = m.v[1];
                w = rsub(e);
            }
        }
        if (small) {
            mac<0>(m0, w);
            if (m1) mac<1>(m1, w);
        } else {
            gen = fr_add(gen, fr_mmul(x, e));
        }
    }
    // T * R^-1 for the unreduced T = lo + hi * 2^256: (lo mod r) * R^-1 + hi
    ZKB_DEV Fr finish() const {
        Fr lo, hi = fr_zero(), one = fr_zero();
#pragma unroll
        for (int i = 0; i < 8; ++i) lo.v[i] = acc[i];
        fe_final_sub(lo);   // 2^256 < 3r: two conditional subtractions make lo canonical
        fe_final_sub(lo);
        hi.v[0] = acc[8]; hi.v[1] = acc[9]; hi.v[2] = acc[10];
        one.v[0] = 1u;
        return fr_add(fr_add(fr_mmul(lo, one), hi), gen);
    }
};

// Up to 32 challenges passed by value as a kernel argument (1 KiB).
struct Challenges {
    Fr u[32];
};

// Grid size for a grid-stride kernel: enough CTAs for `work` items at `per_block`
// each, capped at `waves` resident CTAs per SM times the SM count.
inline unsigned grid_for(size_t work, unsigned per_block, unsigned waves = 8) {
    size_t need = (work + per_block - 1) / per_block;
    size_t cap = (size_t)sm_count() * waves;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}

// Host helper: build the table E[i] = prod_j (bit_j(i) ? u[j] : 1-u[j]) * R for
// i < 2^k in device memory (Montgomery form), u[0] binding the least-significant
// bit.  montmul(x, E[i]) is then the standard-form product x * eq(u, i).
int build_eq_table(const zkb_fr_t* h_u, unsigned k, Fr* d_table, cudaStream_t stream);

// Sum of `n` Fr values already on the device into d_out[0] (one block).
int launch_final_sum(const Fr* d_in, size_t n, Fr* d_out, cudaStream_t stream);

}  // namespace zkb

namespace zkb {

ZKB_DEV Fr fr_load_cg(const Fr* p) {   // L2-coherent load for data written by other CTAs of the same grid
    Fr r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
    uint4 w0 = __ldcg(q), w1 = __ldcg(q + 1);
    r.v[0] = w0.x; r.v[1] = w0.y; r.v[2] = w0.z; r.v[3] = w0.w;
    r.v[4] = w1.x; r.v[5] = w1.y; r.v[6] = w1.z; r.v[7] = w1.w;
    return r;
}

// Grid-wide sum of NS per-thread accumulators without a second launch: every
// CTA stores its block sums, takes a ticket, and the CTA that draws the last
// ticket adds the per-CTA rows and writes out[0..NS).  Slots whose bit is set
// in `fix_mask` are sums of raw Montgomery products (each carrying 1/R^fix_reps) and are
// multiplied by R^2 fix_reps times here.  The ticket is reset for the next launch.  No
// CTA waits on another.
template <int NS>
ZKB_DEV void grid_sum_finish(Fr (&acc)[NS], Fr* __restrict__ partial, unsigned* __restrict__ ticket,
                             Fr* __restrict__ out, unsigned fix_mask, Fr* /* red: kept for the callers' signature */,
                             int fix_reps = 1) {
    __shared__ Fr stage[NS][32];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    // all NS sums move together: one barrier per level instead of two per sum
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        acc[s] = warp_sum(acc[s]);
        if (lane == 0) stage[s][warp] = acc[s];
    }
    __syncthreads();
    for (int s = warp; s < NS; s += nwarps) {
        Fr v = lane < nwarps ? stage[s][lane] : fr_zero();
        v = warp_sum(v);
        if (lane == 0) fr_store(partial + (size_t)blockIdx.x * NS + s, v);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // the CTA that drew the last ticket: one warp per sum over the per-CTA rows
    for (int s = warp; s < NS; s += nwarps) {
        Fr v = fr_zero();
        for (unsigned b = lane; b < gridDim.x; b += 32) v = fr_add(v, fr_load_cg(partial + (size_t)b * NS + s));
        v = warp_sum(v);
        if (lane == 0) {
            if ((fix_mask >> s) & 1u)
                for (int t = 0; t < fix_reps; ++t) v = fr_mmul(v, fe_r2<FrP>());
            fr_store(out + s, v);
        }
    }
    if (threadIdx.x == 0) *ticket = 0;
}

}  // namespace zkb
