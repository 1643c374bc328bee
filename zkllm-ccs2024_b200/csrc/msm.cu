// Pedersen/Hyrax row commitment as a bucket-method multi-scalar multiplication.
//
// Commitment::commit_int (commitment.cu:31-58) multiplies every (scalar,
// generator) pair with a 31-step double-and-add, stores all m*n products and
// tree-sums each row.  Here each row is a Pippenger MSM over the shared
// generator set:
//
//   1. generators are normalised to affine once per call;
//   2. every scalar is split into signed 7-bit digits d_w in [-64, 63] (adding
//      0x40 to every 7-bit field makes each digit an independent bit-field
//      read, no carry chain);  the number of windows follows the largest
//      |scalar| of the call, so 14-bit fixed-point weights need two windows;
//   3. per (row, column segment, window) a counting sort in shared memory
//      groups the non-zero digits by bucket |d|;
//   4. one warp accumulates bucket b of window w for 32 (row, segment) lists at
//      a time with mixed Jacobian+affine additions; the lists of a bucket are
//      ordered by length first, so the lanes of a warp stay in step;
//   5. buckets are combined per row: sum_b b*B_b by running sums over groups
//      of 8 buckets, then Horner over the windows.
//
// The m*n*144-byte product array of the reference is never formed.
#include "comm.cuh"
#include "frutil.cuh"
#include "g1.cuh"
#include "hostfr.hpp"

#include <map>
#include <mutex>
#include <vector>

namespace zkb {

static constexpr int kWinBits = 7;
static constexpr int kBuckets = 64;           // |digit| in 1..64
static constexpr unsigned kMaxSeg = 16384;    // columns per sorted list (u16 entries: col << 1 | neg)
static constexpr int kMaxWindows = 37;        // ceil(259 / 7) for full-width scalars
static constexpr int kGlvWindows = 19;        // ceil(133 / 7): the 128-bit halves of a scalar split by the endomorphism

// ---- digits ------------------------------------------------------------------
// int32 scalar: magnitude + sign; digit w of (|s| + K), K = 0x40 in every field.
ZKB_DEV int digit_of_u64(unsigned long long biased, int w) {
    return (int)((biased >> (kWinBits * w)) & 127u) - 64;
}
__host__ __device__ constexpr unsigned long long bias_u64() {
    unsigned long long k = 0;
    for (int w = 0; w < 9; ++w) k |= 64ull << (kWinBits * w);
    return k;
}

// Full-width scalar: 9-limb (a + K), digit read across limb boundaries.
struct Biased288 { uint32_t l[9]; };
ZKB_DEV Biased288 bias_fr(const Fr& a) {
    // K = 0x40 in each of the 37 seven-bit fields = repeating bit pattern
    Biased288 r;
    uint32_t carry = 0;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
        // limb i of K: bits 32i .. 32i+31; field bit 6 of window w sits at 7w + 6
        uint32_t k = 0;
#pragma unroll
        for (int bit = 0; bit < 32; ++bit) {
            const int pos = 32 * i + bit;
            if (pos % 7 == 6 && pos / 7 < kMaxWindows) k |= 1u << bit;
        }
        const uint32_t ai = i < 8 ? a.v[i] : 0u;
        const unsigned long long s = (unsigned long long)ai + k + carry;
        r.l[i] = (uint32_t)s;
        carry = (uint32_t)(s >> 32);
    }
    return r;
}
ZKB_DEV int digit_of_288(const Biased288& b, int w) {
    const int pos = kWinBits * w, limb = pos >> 5, sh = pos & 31;
    unsigned long long two = b.l[limb];
    if (limb + 1 < 9) two |= (unsigned long long)b.l[limb + 1] << 32;
    return (int)((two >> sh) & 127u) - 64;
}

// ---- kernels -------------------------------------------------------------------
__global__ void i32_absmax_kernel(const int32_t* __restrict__ s, size_t n, unsigned* __restrict__ out) {
    unsigned m = 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int v = s[i];
        const unsigned a = v < 0 ? 0u - (unsigned)v : (unsigned)v;
        m = a > m ? a : m;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned o = __shfl_down_sync(0xffffffffu, m, off);
        m = o > m ? o : m;
    }
    if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

struct MsmShape {
    size_t m, n;          // rows, generators
    unsigned nseg, seg;   // column segments per row and their length
    int W;                // windows
    // Full-width scalars fill only a few buckets of the top window (a 256-bit value has 4 bits there, a 128-bit
    // half 2), so those few lists would be many times longer than all others and one warp would walk them long
    // after the rest of the grid has finished.  The top window therefore spreads every digit over `top_spread`
    // buckets by the low bits of the column: bucket (|d| - 1) * top_spread + (column mod top_spread); a small
    // kernel adds them back into bucket |d| - 1 before the reduction (msm_top_collapse_kernel).  1 = off.
    unsigned top_spread;
};

// bucket 1..64 of a non-zero digit d in window w for column c
ZKB_DEV unsigned bucket_of(const MsmShape& sh, int w, int d, size_t c) {
    const unsigned a = (unsigned)(d < 0 ? -d : d);
    if (sh.top_spread > 1 && w == sh.W - 1) return (a - 1) * sh.top_spread + (unsigned)(c & (sh.top_spread - 1)) + 1;
    return a;
}

// One CTA per (segment, row, window class z): for each of its windows (z, z + gridDim.z, ...),
// counting-sort the non-zero digits of the segment by bucket.  ent: u16 lists, offs: 65 offsets per list.
template <bool FULL>
__global__ void __launch_bounds__(256) msm_sort_kernel(const void* __restrict__ scalars, MsmShape sh,
                                                        uint16_t* __restrict__ ent, uint16_t* __restrict__ offs) {
    extern __shared__ uint16_t list[];           // sh.seg entries
    __shared__ unsigned hist[kBuckets + 1];
    __shared__ unsigned cursor[kBuckets + 1];
    const unsigned seg_id = blockIdx.x;
    const size_t row = blockIdx.y;
    const size_t col0 = (size_t)seg_id * sh.seg;
    const size_t ncol = (col0 + sh.seg <= sh.n) ? sh.seg : (sh.n > col0 ? sh.n - col0 : 0);
    const size_t rs = row * sh.nseg + seg_id;
    for (int w = blockIdx.z; w < sh.W; w += gridDim.z) {
        if (threadIdx.x <= kBuckets) hist[threadIdx.x] = 0;
        __syncthreads();
        for (size_t c = threadIdx.x; c < ncol; c += blockDim.x) {
            int d;
            if (FULL) {
                d = digit_of_288(bias_fr(fr_load(static_cast<const Fr*>(scalars) + row * sh.n + col0 + c)), w);
            } else {
                const int v = static_cast<const int32_t*>(scalars)[row * sh.n + col0 + c];
                const unsigned a = v < 0 ? 0u - (unsigned)v : (unsigned)v;
                d = digit_of_u64((unsigned long long)a + bias_u64(), w);
                if (v < 0) d = -d;
            }
            if (d) atomicAdd(&hist[bucket_of(sh, w, d, c)], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned run = 0;
            uint16_t* o = offs + (rs * sh.W + w) * (kBuckets + 1);
            for (int b = 1; b <= kBuckets; ++b) {
                cursor[b] = run;
                o[b - 1] = (uint16_t)run;
                run += hist[b];
            }
            o[kBuckets] = (uint16_t)run;
        }
        __syncthreads();
        for (size_t c = threadIdx.x; c < ncol; c += blockDim.x) {
            int d;
            if (FULL) {
                d = digit_of_288(bias_fr(fr_load(static_cast<const Fr*>(scalars) + row * sh.n + col0 + c)), w);
            } else {
                const int v = static_cast<const int32_t*>(scalars)[row * sh.n + col0 + c];
                const unsigned a = v < 0 ? 0u - (unsigned)v : (unsigned)v;
                d = digit_of_u64((unsigned long long)a + bias_u64(), w);
                if (v < 0) d = -d;
            }
            if (d) {
                const unsigned pos = atomicAdd(&cursor[bucket_of(sh, w, d, c)], 1u);
                list[pos] = (uint16_t)((c << 1) | (d < 0 ? 1u : 0u));
            }
        }
        __syncthreads();
        uint16_t* e = ent + (rs * sh.W + w) * (size_t)sh.seg;
        const unsigned total = cursor[kBuckets];   // end of the last bucket
        for (unsigned i = threadIdx.x; i < total; i += blockDim.x) e[i] = list[i];
        __syncthreads();
    }
}

// One CTA per (window, bucket): orders the (row, segment) lists of that bucket by
// decreasing length (in bins of 4 entries), so that the 32 lists a warp walks
// in lockstep have nearly the same length and the longest lists start first.
static constexpr unsigned kLenBins = kMaxSeg / 4 + 2;
__global__ void __launch_bounds__(256) msm_schedule_kernel(const uint16_t* __restrict__ offs, MsmShape sh, size_t n_rs,
                                                            uint32_t* __restrict__ perm) {
    __shared__ unsigned hist[kLenBins];
    const unsigned w = blockIdx.x / kBuckets, b = blockIdx.x % kBuckets;
    for (unsigned i = threadIdx.x; i < kLenBins; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (size_t rs = threadIdx.x; rs < n_rs; rs += blockDim.x) {
        const uint16_t* o = offs + (rs * sh.W + w) * (kBuckets + 1);
        atomicAdd(&hist[(unsigned)(o[b + 1] - o[b]) >> 2], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {   // exclusive prefix from the longest bin down
        unsigned run = 0;
        for (int i = (int)kLenBins - 1; i >= 0; --i) {
            const unsigned c = hist[i];
            hist[i] = run;
            run += c;
        }
    }
    __syncthreads();
    uint32_t* out = perm + (size_t)blockIdx.x * n_rs;
    for (size_t rs = threadIdx.x; rs < n_rs; rs += blockDim.x) {
        const uint16_t* o = offs + (rs * sh.W + w) * (kBuckets + 1);
        const unsigned pos = atomicAdd(&hist[(unsigned)(o[b + 1] - o[b]) >> 2], 1u);
        out[pos] = (uint32_t)rs;
    }
}

// One warp per (32 lists of similar length, window, bucket).  blockIdx.x
// enumerates (list group, window, bucket) with the bucket fastest.
// (CTAs of 2 warps or of 1 warp, with the same number of warps per SM, measured 2 to 4 % slower on the opening)
#ifndef ZKB_ACC_WARPS
#define ZKB_ACC_WARPS 4
#endif
static constexpr unsigned kAccWarps = ZKB_ACC_WARPS;
#ifndef ZKB_ACC_MINBLOCKS
#define ZKB_ACC_MINBLOCKS 3
#endif
__global__ void __launch_bounds__(kAccWarps * 32, ZKB_ACC_MINBLOCKS) msm_accumulate_kernel(const G1Aff* __restrict__ bases, MsmShape sh,
                                                                         const uint16_t* __restrict__ ent,
                                                                         const uint16_t* __restrict__ offs,
                                                                         const uint32_t* __restrict__ perm,
                                                                         G1Jac* __restrict__ buckets, size_t n_units) {
    const size_t unit = (size_t)blockIdx.x * kAccWarps + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    const unsigned lane = threadIdx.x & 31;
    const unsigned b = (unsigned)(unit % kBuckets);           // bucket index 0..63 <-> |digit| = b + 1
    const unsigned w = (unsigned)((unit / kBuckets) % sh.W);
    const size_t grp = unit / ((size_t)kBuckets * sh.W);
    const size_t n_rs = sh.m * sh.nseg;
    if (grp * 32 + lane >= n_rs) return;
    const size_t rs = perm[((size_t)w * kBuckets + b) * n_rs + grp * 32 + lane];
    const size_t list_id = rs * sh.W + w;
    const uint16_t* o = offs + list_id * (kBuckets + 1);
    const unsigned beg = o[b], end = o[b + 1];
    const uint16_t* e = ent + list_id * (size_t)sh.seg;
    const size_t col0 = (rs % sh.nseg) * (size_t)sh.seg;
#ifdef ZKB_ACC_JACOBIAN
    G1Jac acc = g1_identity();
    for (unsigned i = beg; i < end; ++i) {
        const unsigned code = e[i];
        G1Aff p = g1_aff_load(bases + col0 + (code >> 1));
        if (code & 1u) p = g1_aff_neg(p);
        acc = g1_add_mixed(acc, p);
    }
    g1_store(buckets + list_id * kBuckets + b, acc);
#else
    G1Xyzz acc = xyzz_identity();                 // 10 products per mixed addition (11 in Jacobian coordinates)
    for (unsigned i = beg; i < end; ++i) {
        const unsigned code = e[i];
        G1Aff p = g1_aff_load(bases + col0 + (code >> 1));
        if (code & 1u) p = g1_aff_neg(p);
        acc = xyzz_add_mixed(acc, p);
    }
    g1_store(buckets + list_id * kBuckets + b, xyzz_to_jac(acc));
#endif
}

// One CTA of 64 threads per (row, segment) list: the spread buckets of the top window (MsmShape::top_spread)
// added back into bucket |d| - 1, the others cleared.
__global__ void __launch_bounds__(64) msm_top_collapse_kernel(G1Jac* __restrict__ buckets, MsmShape sh) {
    const size_t list_id = (size_t)blockIdx.x * sh.W + (sh.W - 1);
    G1Jac* b = buckets + list_id * kBuckets;
    const unsigned F = sh.top_spread, j = threadIdx.x;
    G1Jac sum = g1_identity();
    if (j < kBuckets / F)
        for (unsigned t = 0; t < F; ++t) sum = g1_add(sum, g1_load(b + j * F + t));
    __syncthreads();
    g1_store(b + j, sum);
}

// Thread per (row, window, group of 8 buckets): sums the segment partials of its
// buckets and forms the group's running sums.
//   Lg[(row*W + w)*8 + g] = sum_{i=1..8} i * B_{8g+i}      Gg[...] = sum_i B_{8g+i}
__global__ void __launch_bounds__(128) msm_group_kernel(const G1Jac* __restrict__ buckets, MsmShape sh,
                                                         G1Jac* __restrict__ Lg, G1Jac* __restrict__ Gg) {
    const size_t total = sh.m * sh.W * 8;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const unsigned g = (unsigned)(t & 7);
        const unsigned w = (unsigned)((t >> 3) % sh.W);
        const size_t row = (t >> 3) / sh.W;
        G1Jac run = g1_identity(), loc = g1_identity();
        for (int i = 8; i >= 1; --i) {
            const unsigned b = 8 * g + i - 1;
            for (unsigned s = 0; s < sh.nseg; ++s) {
                const size_t list_id = (row * sh.nseg + s) * sh.W + w;
                run = g1_add(run, g1_load(buckets + list_id * kBuckets + b));
            }
            loc = g1_add(loc, run);
        }
        g1_store(Lg + t, loc);
        g1_store(Gg + t, run);
    }
}

// Thread per row: window sums from the group results, then Horner over windows.
__global__ void __launch_bounds__(128) msm_finish_kernel(const G1Jac* __restrict__ Lg, const G1Jac* __restrict__ Gg,
                                                          MsmShape sh, G1Jac* __restrict__ out) {
    for (size_t row = blockIdx.x * (size_t)blockDim.x + threadIdx.x; row < sh.m; row += (size_t)gridDim.x * blockDim.x) {
        G1Jac acc = g1_identity();
        for (int w = sh.W - 1; w >= 0; --w) {
            if (w != sh.W - 1) {
                for (int d = 0; d < kWinBits; ++d) acc = g1_double(acc);
            }
            const size_t base = (row * sh.W + w) * 8;
            // window total = sum_g Lg + 8 * sum_{g>=1} g * Gg
            G1Jac lsum = g1_identity(), run = g1_identity(), t = g1_identity();
            for (int g = 7; g >= 0; --g) {
                lsum = g1_add(lsum, g1_load(Lg + base + g));
                if (g >= 1) {
                    run = g1_add(run, g1_load(Gg + base + g));
                    t = g1_add(t, run);
                }
            }
            t = g1_double(g1_double(g1_double(t)));
            acc = g1_add(acc, g1_add(lsum, t));
        }
        g1_store(out + row, acc);
    }
}

// Jacobian -> affine with one field inversion per thread shared by `per_thread`
// points (Montgomery's trick).  A block owns blockDim.x * per_thread consecutive
// points; thread t takes t, t + blockDim.x, ...  The running prefix product of
// the z coordinates is parked in out[i].x until the way back.
__global__ void __launch_bounds__(128) g1_to_affine_batched_kernel(const G1Jac* __restrict__ a, G1Aff* __restrict__ out, size_t n,
                                                                    unsigned per_thread) {
    const size_t tile0 = (size_t)blockIdx.x * blockDim.x * per_thread + threadIdx.x;
    Fq acc = fe_mont_one<FqParams>();
    for (unsigned j = 0; j < per_thread; ++j) {
        const size_t i = tile0 + (size_t)j * blockDim.x;
        if (i >= n) break;
        const Fq z = fe_load(&a[i].z);
        fe_store(&out[i].x, acc);
        if (!fe_is_zero(z)) acc = fq_mul(acc, z);
    }
    Fq inv = mont_inv<FqParams>(acc);
    for (int j = (int)per_thread - 1; j >= 0; --j) {
        const size_t i = tile0 + (size_t)j * blockDim.x;
        if (i >= n) continue;
        const G1Jac p = g1_load(a + i);
        G1Aff r;
        if (g1_is_identity(p)) {
            r.x = fe_zero<FqParams>(); r.y = fe_zero<FqParams>();
        } else {
            const Fq zi = fq_mul(inv, fe_load(&out[i].x));
            inv = fq_mul(inv, p.z);
            const Fq zi2 = fq_sqr(zi);
            r.x = fq_mul(p.x, zi2);
            r.y = fq_mul(p.y, fq_mul(zi2, zi));
        }
        g1_aff_store(out + i, r);
    }
}

static int to_affine_device(const G1Jac* d_a, G1Aff* d_out, size_t n, cudaStream_t s) {
    if (n == 0) return ZKB_OK;
    size_t per_thread = n / 32768;
    if (per_thread < 1) per_thread = 1;
    if (per_thread > 32) per_thread = 32;
    const size_t tile = 128 * per_thread;
    ZKB_LAUNCH(g1_to_affine_batched_kernel, (unsigned)((n + tile - 1) / tile), 128, 0, s, d_a, d_out, n, (unsigned)per_thread);
    return ZKB_OK;
}

// ---- few rows, many windows: bucket partials are first summed over the segments,
// then every (row, window) total is formed in parallel and one thread per row
// runs Horner over the windows. -----------------------------------------------------
// Block of 128 threads = 16 buckets x 8 segment parts.  red[(row*W + w)*64 + b].
__global__ void __launch_bounds__(128) msm_seg_reduce_kernel(const G1Jac* __restrict__ buckets, MsmShape sh, G1Jac* __restrict__ red) {
    __shared__ G1Jac sm[128];
    const unsigned part = threadIdx.x & 7, bl = threadIdx.x >> 3;
    const size_t rwq = blockIdx.x;                     // (row*W + w)*4 + quarter
    const unsigned b = (unsigned)(rwq & 3) * 16 + bl;
    const unsigned w = (unsigned)((rwq >> 2) % sh.W);
    const size_t row = (rwq >> 2) / sh.W;
    G1Jac acc = g1_identity();
    for (unsigned sg = part; sg < sh.nseg; sg += 8) {
        const size_t list_id = (row * sh.nseg + sg) * sh.W + w;
        acc = g1_add(acc, g1_load(buckets + list_id * kBuckets + b));
    }
    sm[threadIdx.x] = acc;
    __syncthreads();
    for (unsigned step = 4; step > 0; step >>= 1) {
        if (part < step) sm[threadIdx.x] = g1_add(sm[threadIdx.x], sm[threadIdx.x + step]);
        __syncthreads();
    }
    if (part == 0) g1_store(red + (rwq >> 2) * kBuckets + b, sm[threadIdx.x]);
}

// Thread per (row, window): total of the window from its eight group results.
__global__ void __launch_bounds__(64) msm_window_kernel(const G1Jac* __restrict__ Lg, const G1Jac* __restrict__ Gg, size_t n_rw,
                                                         G1Jac* __restrict__ win) {
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n_rw; t += (size_t)gridDim.x * blockDim.x) {
        const size_t base = t * 8;
        G1Jac lsum = g1_identity(), run = g1_identity(), acc = g1_identity();
        for (int g = 7; g >= 0; --g) {
            lsum = g1_add(lsum, g1_load(Lg + base + g));
            if (g >= 1) {
                run = g1_add(run, g1_load(Gg + base + g));
                acc = g1_add(acc, run);
            }
        }
        acc = g1_double(g1_double(g1_double(acc)));
        g1_store(win + t, g1_add(lsum, acc));
    }
}

__global__ void __launch_bounds__(32) msm_horner_kernel(const G1Jac* __restrict__ win, MsmShape sh, G1Jac* __restrict__ out) {
    for (size_t row = blockIdx.x * (size_t)blockDim.x + threadIdx.x; row < sh.m; row += (size_t)gridDim.x * blockDim.x) {
        G1Jac acc = g1_load(win + row * sh.W + (sh.W - 1));
        for (int w = sh.W - 2; w >= 0; --w) {
            for (int d = 0; d < kWinBits; ++d) acc = g1_double(acc);
            acc = g1_add(acc, g1_load(win + row * sh.W + w));
        }
        g1_store(out + row, acc);
    }
}

// Shape of one MSM call: enough (row, segment) lists to fill warps, segments no
// longer than kMaxSeg.  One list group of 32 lanes gives W * 64 warps, so
// full-width scalars need only a few groups and prefer long lists; small integers
// need thousands.  nseg_fixed != 0 prescribes the segment count (callers that
// put the buckets of several calls into one array for a common reduction).
static int msm_shape(size_t n, size_t m, int W, bool full, size_t nseg_fixed, MsmShape* out) {
    MsmShape sh;
    sh.m = m; sh.n = n; sh.W = W;
    // full-width scalars come with few rows: enough (row, segment) lists for about 7000 warps of 32 lists per
    // (window, bucket) - twice as many segments for the 19 windows of the endomorphism split as for 37
    const size_t want_lists = full ? (W <= kGlvWindows ? 192 : 96) : 4096;
    size_t nseg = (want_lists + m - 1) / m;
    const size_t min_seg_len = full ? 64 : 256;
    if (nseg > (n + min_seg_len - 1) / min_seg_len) nseg = (n + min_seg_len - 1) / min_seg_len;
    if (nseg < (n + kMaxSeg - 1) / kMaxSeg) nseg = (n + kMaxSeg - 1) / kMaxSeg;
    if (nseg < 1) nseg = 1;
    if (nseg_fixed) {
        if (nseg_fixed < (n + kMaxSeg - 1) / kMaxSeg) return fail(ZKB_ERR_LIMIT, "commit: prescribed segment count too small");
        nseg = nseg_fixed;
    }
    if (nseg > 65535) return fail(ZKB_ERR_LIMIT, "commit: more than 2^30 generators");
    if (m > 65535 * 32) return fail(ZKB_ERR_LIMIT, "commit: too many rows");
    if (m * nseg > 0xffffffffull) return fail(ZKB_ERR_LIMIT, "commit: too many (row, segment) lists");
    sh.nseg = (unsigned)nseg;
    sh.seg = (unsigned)((n + nseg - 1) / nseg);
    // the top digit of a 256-bit scalar in 37 windows is at most 16, of a 128-bit half in 19 windows at most 4
    sh.top_spread = !full ? 1u : (W == kMaxWindows ? 4u : (W == kGlvWindows ? 16u : 1u));
    *out = sh;
    return ZKB_OK;
}
static size_t msm_bucket_count(const MsmShape& sh) { return sh.m * sh.nseg * (size_t)sh.W * kBuckets; }

// Phase 1: digits -> sorted lists -> bucket sums per (row, segment, window), into
// `buckets` (msm_bucket_count entries).  `scalars` is int32[m*n] (FULL = false) or
// raw 256-bit Fr limbs [m*n] (FULL = true).
template <bool FULL>
static int msm_accumulate_phase(const G1Aff* bases, const void* d_scalars, const MsmShape& sh, G1Jac* buckets,
                                Scratch& scratch, cudaStream_t s) {
    const size_t m = sh.m, n = sh.n, nseg = sh.nseg;
    const int W = sh.W;
    const size_t n_rs = m * nseg;
    const size_t n_lists = n_rs * W;
    uint16_t* ent = scratch.get_n<uint16_t>(n_lists * sh.seg);
    uint16_t* offs = scratch.get_n<uint16_t>(n_lists * (kBuckets + 1));
    uint32_t* perm = scratch.get_n<uint32_t>((size_t)W * kBuckets * n_rs);
    if (!ent || !offs || !perm) return ZKB_ERR_CUDA;
    // full-width scalars: few lists, many windows -> one CTA per (segment, row, window)
    const unsigned zdim = FULL ? (unsigned)W : 1u;
    // rows go to gridDim.y in slices of at most 65535
    for (size_t r0 = 0; r0 < m; r0 += 65535) {
        const size_t rows = (m - r0 < 65535) ? m - r0 : 65535;
        MsmShape part = sh;
        part.m = rows;
        const void* sc = FULL ? static_cast<const void*>(static_cast<const Fr*>(d_scalars) + r0 * n)
                              : static_cast<const void*>(static_cast<const int32_t*>(d_scalars) + r0 * n);
        ZKB_LAUNCH(msm_sort_kernel<FULL>, dim3(sh.nseg, (unsigned)rows, zdim), 256, sh.seg * sizeof(uint16_t), s,
                   sc, part, ent + r0 * nseg * W * sh.seg, offs + r0 * nseg * W * (kBuckets + 1));
    }
    const size_t n_groups = (n_rs + 31) / 32;
    const size_t n_units = n_groups * W * kBuckets;
    const size_t acc_blocks = (n_units + kAccWarps - 1) / kAccWarps;
    if (acc_blocks > 0x7fffffffull) return fail(ZKB_ERR_LIMIT, "commit: problem too large for one launch");
    ZKB_LAUNCH(msm_schedule_kernel, (unsigned)(W * kBuckets), 256, 0, s, offs, sh, n_rs, perm);
    ZKB_LAUNCH(msm_accumulate_kernel, (unsigned)acc_blocks, kAccWarps * 32, 0, s, bases, sh, ent, offs, perm, buckets, n_units);
    return ZKB_OK;
}

// Phase 2: bucket sums -> one point per row.  Only m, nseg and W of the shape are used,
// so the buckets of several phase-1 calls with equal nseg and W reduce together.
static int msm_reduce_phase(G1Jac* buckets, const MsmShape& sh, G1Jac* d_out, Scratch& scratch, cudaStream_t s) {
    const size_t m = sh.m;
    const int W = sh.W;
    if (sh.top_spread > 1) {
        if (m * sh.nseg > 0x7fffffffull) return fail(ZKB_ERR_LIMIT, "commit: too many (row, segment) lists");
        ZKB_LAUNCH(msm_top_collapse_kernel, (unsigned)(m * sh.nseg), 64, 0, s, buckets, sh);
    }
    G1Jac* Lg = scratch.get_n<G1Jac>(m * W * 8);
    G1Jac* Gg = scratch.get_n<G1Jac>(m * W * 8);
    if (!Lg || !Gg) return ZKB_ERR_CUDA;
    if (m * W >= 4096) {
        ZKB_LAUNCH(msm_group_kernel, grid_for(m * W * 8, 128), 128, 0, s, buckets, sh, Lg, Gg);
        ZKB_LAUNCH(msm_finish_kernel, grid_for(m, 128), 128, 0, s, Lg, Gg, sh, d_out);
        return ZKB_OK;
    }
    // few rows: sum over the segments first, all window totals in parallel, one Horner thread per row
    G1Jac* win = scratch.get_n<G1Jac>(m * W);
    if (!win) return ZKB_ERR_CUDA;
    const G1Jac* src = buckets;
    MsmShape one = sh;
    if (sh.nseg > 1) {
        G1Jac* red = scratch.get_n<G1Jac>(m * W * kBuckets);
        if (!red) return ZKB_ERR_CUDA;
        ZKB_LAUNCH(msm_seg_reduce_kernel, (unsigned)(m * W * 4), 128, 0, s, buckets, sh, red);
        src = red;
        one.nseg = 1;   // `red` is laid out like the bucket array of a single segment
    }
    ZKB_LAUNCH(msm_group_kernel, grid_for(m * W * 8, 64), 64, 0, s, src, one, Lg, Gg);
    ZKB_LAUNCH(msm_window_kernel, grid_for(m * W, 64), 64, 0, s, Lg, Gg, m * W, win);
    ZKB_LAUNCH(msm_horner_kernel, grid_for(m, 32), 32, 0, s, win, sh, d_out);
    return ZKB_OK;
}

template <bool FULL>
static int msm_rows_affine(const G1Aff* bases, size_t n, const void* d_scalars, size_t m, int W,
                           G1Jac* d_out, Scratch& scratch, cudaStream_t s) {
    if (m == 0) return ZKB_OK;
    MsmShape sh;
    ZKB_TRY(msm_shape(n, m, W, FULL, 0, &sh));
    G1Jac* buckets = scratch.get_n<G1Jac>(msm_bucket_count(sh));
    if (!buckets) return ZKB_ERR_CUDA;
    ZKB_TRY(msm_accumulate_phase<FULL>(bases, d_scalars, sh, buckets, scratch, s));
    return msm_reduce_phase(buckets, sh, d_out, scratch, s);
}

// The same over Jacobian generators: normalised to affine once per call.
template <bool FULL>
static int msm_rows(const G1Jac* d_gens, size_t n, const void* d_scalars, size_t m, int W,
                    G1Jac* d_out, Scratch& scratch, cudaStream_t s) {
    if (m == 0) return ZKB_OK;
    G1Aff* bases = scratch.get_n<G1Aff>(n);
    if (!bases) return ZKB_ERR_CUDA;
    ZKB_TRY(to_affine_device(d_gens, bases, n, s));
    return msm_rows_affine<FULL>(bases, n, d_scalars, m, W, d_out, scratch, s);
}

// ---- full-width scalars over points of order r, through the endomorphism -------------------
// phi(x, y) = (beta x, y) = [lambda] (x, y) on the order-r group, lambda = z^2 - 1 (128 bits).  A scalar k (raw
// 256-bit limbs, any value) is reduced modulo r and written k = k1 + k2 lambda with k1 < lambda, k2 < 2^128, and
// k P = k1 P + k2 phi(P): an MSM over n points with 255-bit scalars becomes one over 2n points with 128-bit
// scalars.  The bucket additions stay the same (2 x 19 windows for 37), but the per-window sums, their
// reduction and the doublings of the final Horner pass (the longest dependent chain of a small MSM) halve.
// Only zkb_me_open's fast path uses it, after its generators passed the order check.

ZKB_DEV void glv_split(const Fr& raw, Fr& k1, Fr& k2) {
    typedef unsigned __int128 u128;
    const u128 lambda = ((u128)0xac45a4010001a402ull << 64) | 0x00000000ffffffffull;
    const uint64_t rmod[4] = {0xffffffff00000001ull, 0x53bda402fffe5bfeull, 0x3339d80809a1d805ull, 0x73eda753299d7d48ull};
    uint64_t limb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) limb[i] = ((uint64_t)raw.v[2 * i + 1] << 32) | raw.v[2 * i];
    k1 = fr_zero();
    k2 = fr_zero();
    if ((limb[0] | limb[1] | limb[2] | limb[3]) == 0) return;
    for (int pass = 0; pass < 2; ++pass) {          // 2^256 < 3 r
        bool ge = true;
        for (int i = 3; i >= 0; --i)
            if (limb[i] != rmod[i]) { ge = limb[i] > rmod[i]; break; }
        if (!ge) break;
        uint64_t borrow = 0;
        for (int i = 0; i < 4; ++i) {
            const u128 d = (u128)limb[i] - rmod[i] - borrow;
            limb[i] = (uint64_t)d;
            borrow = (uint64_t)(d >> 64) ? 1 : 0;
        }
    }
    u128 rem = 0, quo = 0;                           // schoolbook division by lambda, one bit at a time
#pragma unroll 1
    for (int bit = 255; bit >= 0; --bit) {
        const bool top = (bool)(rem >> 127);
        rem = (rem << 1) | ((limb[bit >> 6] >> (bit & 63)) & 1u);
        quo <<= 1;
        if (top || rem >= lambda) { rem -= lambda; quo |= 1; }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        k1.v[i] = (uint32_t)(rem >> (32 * i));
        k2.v[i] = (uint32_t)(quo >> (32 * i));
    }
}

__global__ void __launch_bounds__(256) glv_rows_kernel(const Fr* __restrict__ rows, size_t total, Fr* __restrict__ out) {
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        Fr k1, k2;
        glv_split(fr_load(rows + e), k1, k2);
        fr_store(out + 2 * e, k1);
        fr_store(out + 2 * e + 1, k2);
    }
}

// beta: the cube root of unity in Fq that goes with lambda (Montgomery form)
ZKB_DEV Fq fq_beta_mont() {
    constexpr uint32_t t[12] = {0x8671f071u, 0xcd03c9e4u, 0x1fcda5d2u, 0x5dab2246u, 0xd3851b95u, 0x587042afu,
                                0x01bacb9eu, 0x8eb60ebeu, 0x83d050d2u, 0x03f97d6eu, 0x54638741u, 0x18f02065u};
    Fq r;
#pragma unroll
    for (int i = 0; i < 12; ++i) r.v[i] = t[i];
    return r;
}
__global__ void __launch_bounds__(256) glv_bases_kernel(const G1Aff* __restrict__ bases, size_t n, G1Aff* __restrict__ out) {
    const Fq beta = fq_beta_mont();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        G1Aff p = g1_aff_load(bases + i);
        g1_aff_store(out + 2 * i, p);
        p.x = fq_mul(p.x, beta);                     // the affine identity (0, 0) stays what it is
        g1_aff_store(out + 2 * i + 1, p);
    }
}

// bases2: 2n points, rows2: m x 2n scalars for msm_*<true> with kGlvWindows windows
static int glv_expand(const G1Aff* bases, size_t n, const Fr* d_rows, size_t m, G1Aff** bases2, Fr** rows2,
                      Scratch& scratch, cudaStream_t s) {
    *bases2 = scratch.get_n<G1Aff>(2 * n);
    *rows2 = scratch.get_n<Fr>(2 * m * n);
    if (!*bases2 || !*rows2) return ZKB_ERR_CUDA;
    ZKB_LAUNCH(glv_bases_kernel, grid_for(n, 256), 256, 0, s, bases, n, *bases2);
    ZKB_LAUNCH(glv_rows_kernel, grid_for(m * n, 256), 256, 0, s, d_rows, m * n, *rows2);
    return ZKB_OK;
}

static int msm_rows_affine_glv(const G1Aff* bases, size_t n, const Fr* d_rows, size_t m, G1Jac* d_out, Scratch& scratch,
                               cudaStream_t s) {
    if (m == 0) return ZKB_OK;
    G1Aff* b2 = nullptr;
    Fr* r2 = nullptr;
    ZKB_TRY(glv_expand(bases, n, d_rows, m, &b2, &r2, scratch, s));
    return msm_rows_affine<true>(b2, 2 * n, r2, m, kGlvWindows, d_out, scratch, s);
}

// Smallest W such that |s| + K stays below 128^W for every |s| <= max_abs, where
// K is 0x40 in each of the W fields: max_abs < (63 * 128^W + 64) / 127.
static int windows_for_max(unsigned long long max_abs) {
    unsigned long long p = 128;
    for (int W = 1; W < 9; ++W, p *= 128)
        if (max_abs * 127 < 63 * p + 64) return W;
    return 9;
}

}  // namespace zkb
#include "msm_comb.cuh"
namespace zkb {

// Field products of the bucket method for m rows (unit shared with comb_cost).
static double bucket_cost(size_t m, size_t n, int W) {
    return (double)m * W * ((double)n * 11.0 + 2.0 * kBuckets * 16.0);
}

// int32 path: find the largest magnitude (one small D2H), then either the bucket
// method with 7-bit windows or, for many rows over one generator set, the
// combination tables of msm_comb.cuh with 3-bit windows - whichever needs fewer field
// products.  method: ZKB_MSM_AUTO, or one of the two by name.
static constexpr size_t kCombTableLimit = (size_t)12 << 30;
// early_table: tables of this generator set that the caller built while the scalars were still being copied
// (zkb_commit_i32_host), or nullptr.
static int commit_i32_device(const G1Jac* d_gens, size_t n_gen, const int32_t* d_scalars, size_t n_scalars,
                             G1Jac* d_out, Scratch& scratch, cudaStream_t s, int method = ZKB_MSM_AUTO,
                             const G1Aff* early_table = nullptr) {
    if (n_gen == 0 || n_scalars % n_gen) return fail(ZKB_ERR_DIM, "Commitment::commit_int - Incompatible dimensions");
    if (method != ZKB_MSM_AUTO && method != ZKB_MSM_BUCKETS && method != ZKB_MSM_TABLES)
        return fail(ZKB_ERR_ARG, "commit: unknown method");
    const size_t m = n_scalars / n_gen;
    if (m == 0) return ZKB_OK;
    unsigned* d_max = scratch.get_n<unsigned>(4);
    if (!d_max) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemsetAsync(d_max, 0, 16, s));
    ZKB_LAUNCH(i32_absmax_kernel, grid_for(n_scalars, 256 * 8), 256, 0, s, d_scalars, n_scalars, d_max);
    unsigned h_max = 0;
    ZKB_CUDA(cudaMemcpyAsync(&h_max, d_max, 4, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    const int W7 = windows_for_max(h_max), W3 = comb_windows_for_max(h_max);
    bool tables = method == ZKB_MSM_TABLES;
    if (method == ZKB_MSM_AUTO)
        tables = comb_table_bytes(n_gen) <= kCombTableLimit && comb_cost(m, n_gen, W3) < bucket_cost(m, n_gen, W7);
    if (!tables) return msm_rows<false>(d_gens, n_gen, d_scalars, m, W7, d_out, scratch, s);
    if (early_table) return msm_comb_run(early_table, n_gen, d_scalars, m, W3, d_out, scratch, s);
    G1Aff* bases = scratch.get_n<G1Aff>(n_gen);
    if (!bases) return ZKB_ERR_CUDA;
    ZKB_TRY(to_affine_device(d_gens, bases, n_gen, s));
    return msm_comb_rows(bases, n_gen, d_scalars, m, W3, d_out, scratch, s);
}

// ---- opening rounds (Commitment::me_open / me_open_step, commitment.cu:79-125) ----
// Round with scalars s and generators g, both of length `old`, pairs (2j, 2j+1):
//   T  = sum_i s_i g_i     T0 = sum_j s_2j g_2j+1     T1 = sum_j s_2j+1 g_2j
//   s'_j = s_2j + u (s_2j+1 - s_2j)          g'_j = g_2j+1 + u (g_2j - g_2j+1)
// The reference forms five scalar products per pair and tree-sums three arrays.
// Here T, T0, T1 are one three-row MSM over the round's generators (rows 1 and 2
// are the pair-swapped scalars with every other entry zero), which leaves one
// scalar product per pair, for g'.  Scalars are used by their raw limbs, as the
// reference's G1Jacobian_mul reads them.  A lone last element pairs with nothing.
// with_T = 0 leaves the T row out: rows = [T0, T1] (the caller derives T from the round before).
__global__ void me_open_rows_kernel(const Fr* __restrict__ sc, size_t old_size, size_t new_size, Fr u_mont, unsigned with_T,
                                    Fr* __restrict__ rows, Fr* __restrict__ nsc) {
    const Fr zero = fr_zero();
    Fr* row_T0 = rows + (with_T ? old_size : 0);
    Fr* row_T1 = row_T0 + old_size;
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < new_size; g += (size_t)gridDim.x * blockDim.x) {
        const size_t i0 = 2 * g, i1 = 2 * g + 1;
        const Fr s0 = fr_load(sc + i0);
        if (with_T) fr_store(rows + i0, s0);
        fr_store(row_T0 + i0, zero);
        if (i1 >= old_size) {
            fr_store(row_T1 + i0, zero);
            fr_store(nsc + g, fr_sub(s0, fr_mmul(u_mont, s0)));
            continue;
        }
        const Fr s1 = fr_load(sc + i1);
        if (with_T) fr_store(rows + i1, s1);
        fr_store(row_T0 + i1, s0);        // T0: s_2j on g_2j+1
        fr_store(row_T1 + i0, s1);        // T1: s_2j+1 on g_2j
        fr_store(row_T1 + i1, zero);
        fr_store(nsc + g, fr_add(s0, fr_mmul(u_mont, fr_sub(s1, s0))));
    }
}

ZKB_DEV G1Jac g1_from_aff(const G1Aff& a) {
    G1Jac r;
    r.x = a.x; r.y = a.y;
    r.z = g1_aff_is_identity(a) ? fe_zero<FqParams>() : fe_mont_one<FqParams>();
    return r;
}

// u * P for the one scalar u all pairs of a round share, through the curve's
// endomorphism phi(x, y) = (beta x, y) = lambda (x, y) on the order-r group:
// u = k1 + k2 lambda with 128-bit halves (host: fold_digits), both halves in width-5
// non-adjacent form (odd digits -15..15, on average one non-zero digit in six), and
// k1 P + k2 phi(P) by one pass over the bits of both halves with a table of P, 3P, .. 15P:
// 130 doublings and about 43 additions instead of 255 and ~128.  The digits are the same
// for every thread, so the pass does not diverge.
struct FoldDigits { signed char d1[130], d2[130]; };

__device__ __noinline__ static G1Jac g1_add_call(const G1Jac& p, const G1Jac& q) { return g1_add(p, q); }
__device__ __noinline__ static G1Jac g1_double_call(const G1Jac& p) { return g1_double(p); }

__device__ static G1Jac g1_mul_shared_scalar(const G1Jac& p, const FoldDigits& dg) {
    if (g1_is_identity(p)) return p;
    G1Jac tab[8];                                   // (2j + 1) P
    tab[0] = p;
    const G1Jac p2 = g1_double_call(p);
#pragma unroll 1
    for (int j = 1; j < 8; ++j) tab[j] = g1_add_call(tab[j - 1], p2);
    const Fq beta = fq_beta_mont();
    G1Jac acc = g1_identity();
#pragma unroll 1
    for (int i = 129; i >= 0; --i) {
        acc = g1_double_call(acc);
        const int a = dg.d1[i], b = dg.d2[i];
        if (a) {
            G1Jac t = tab[((a < 0 ? -a : a) - 1) >> 1];
            if (a < 0) t = g1_neg(t);
            acc = g1_add_call(acc, t);
        }
        if (b) {
            G1Jac t = tab[((b < 0 ? -b : b) - 1) >> 1];
            t.x = fq_mul(t.x, beta);
            if (b < 0) t = g1_neg(t);
            acc = g1_add_call(acc, t);
        }
    }
    return acc;
}

// Measured on 2^19 generators, the fold alone with 128 threads per CTA: 2 CTAs per SM (214 registers) 51 ms, 3 CTAs (168)
// 59 ms, 4 CTAs 64 ms; an affine table with mixed additions and a non-inlined field product changed nothing.  The same
// 8 warps per SM as 4 CTAs of 64 threads (218 registers) finish a whole opening 2.5 % sooner (86.6 against 88.8 ms).
#ifndef ZKB_FOLD_MINBLOCKS
#define ZKB_FOLD_MINBLOCKS 4
#endif
#ifndef ZKB_FOLD_THREADS
#define ZKB_FOLD_THREADS 64
#endif
__global__ void __launch_bounds__(ZKB_FOLD_THREADS, ZKB_FOLD_MINBLOCKS) me_open_fold_kernel(const G1Aff* __restrict__ bases, size_t old_size, size_t new_size,
                                                            FoldDigits dg, G1Jac* __restrict__ ngen) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < new_size; g += (size_t)gridDim.x * blockDim.x) {
        const G1Aff a0 = g1_aff_load(bases + 2 * g);
        if (2 * g + 1 >= old_size) {
            g1_store(ngen + g, g1_mul_shared_scalar(g1_from_aff(a0), dg));
            continue;
        }
        const G1Aff a1 = g1_aff_load(bases + 2 * g + 1);
        const G1Jac diff = g1_add_mixed(g1_from_aff(a0), g1_aff_neg(a1));
        g1_store(ngen + g, g1_add_mixed(g1_mul_shared_scalar(diff, dg), a1));
    }
}

// Host: u (standard form, below r) = k1 + k2 * lambda, then the width-5 non-adjacent form of both halves.
static FoldDigits fold_digits(const zkb_fr_t& u) {
    typedef unsigned __int128 u128;
    const u128 lambda = ((u128)0xac45a4010001a402ull << 64) | 0x00000000ffffffffull;
    // schoolbook long division of the 256-bit u by lambda, one bit at a time
    uint64_t limb[4];
    for (int i = 0; i < 4; ++i) limb[i] = ((uint64_t)u.val[2 * i + 1] << 32) | u.val[2 * i];
    // a raw value of r or more names the same multiple as its residue (2^256 < 3r)
    const uint64_t rmod[4] = {0xffffffff00000001ull, 0x53bda402fffe5bfeull, 0x3339d80809a1d805ull, 0x73eda753299d7d48ull};
    for (int pass = 0; pass < 2; ++pass) {
        bool ge = true;
        for (int i = 3; i >= 0; --i)
            if (limb[i] != rmod[i]) { ge = limb[i] > rmod[i]; break; }
        if (!ge) break;
        u128 borrow = 0;
        for (int i = 0; i < 4; ++i) {
            const u128 d = (u128)limb[i] - rmod[i] - borrow;   // wraps modulo 2^128 when negative
            limb[i] = (uint64_t)d;
            borrow = (d >> 64) ? 1 : 0;
        }
    }
    u128 rem = 0, quo = 0;
    for (int bit = 255; bit >= 0; --bit) {
        const bool top = (bool)(rem >> 127);
        rem = (rem << 1) | ((limb[bit >> 6] >> (bit & 63)) & 1u);
        quo <<= 1;                         // the quotient of a value below r fits 128 bits
        if (top || rem >= lambda) { rem -= lambda; quo |= 1; }
    }
    FoldDigits out;
    u128 k[2] = {rem, quo};
    for (int h = 0; h < 2; ++h) {
        signed char* d = h ? out.d2 : out.d1;
        u128 v = k[h];
        for (int i = 0; i < 130; ++i) {              // width-5 non-adjacent form, least significant digit first
            int x = 0;
            if (v & 1u) {
                x = (int)(v & 31u);
                if (x >= 16) { x -= 32; v += (u128)(-x); }   // v < 2^128 - 31 here: lambda and the quotient are below 2^128 - 2^125
                else v -= (u128)x;
            }
            d[i] = (signed char)x;
            v >>= 1;
        }
    }
    return out;
}

// ---- generators outside the order-r subgroup ---------------------------------------
// The shortcuts of the opening (endomorphism fold, T rows derived from earlier proof points, the tail as one
// MSM) multiply scalars modulo r, which is the same group element only for points of order r - what
// Commitment::random makes (commitment.cu:3-8), but not what an arbitrary generator file has to hold.  Every
// generator set is therefore checked once; the verdict is kept under a fingerprint of the set.  A set that fails
// takes the reference's own arithmetic (me_open_step, commitment.cu:79-109): three MSM rows in every round, the
// fold as a plain double-and-add by the challenge's 256 raw bits, every round folded.
//
// The check is the endomorphism test of BLS12 curves (M. Scott, "A note on group membership tests for G1, G2 and
// GT on BLS pairing-friendly curves", 2021): with the curve parameter z (r = z^4 - z^2 + 1) a curve point P has
// order r exactly when phi(P) = [z^2 - 1] P, written here as phi(P) + P = [|z|] [|z|] P.  |z| = 0xd201000000010000
// has six bits set, so a point costs 126 doublings and 12 additions instead of the 255 and ~70 of [r] P = O.
__device__ static G1Jac g1_mul_abs_z(const G1Jac& p) {
    constexpr unsigned long long kAbsZ = 0xd201000000010000ull;
    G1Jac acc = p;
#pragma unroll 1
    for (int b = 62; b >= 0; --b) {
        acc = g1_double_call(acc);
        if ((kAbsZ >> b) & 1ull) acc = g1_add_call(acc, p);
    }
    return acc;
}

__global__ void __launch_bounds__(128) g1_order_check_kernel(const G1Jac* __restrict__ gens, size_t n, unsigned* __restrict__ bad) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const G1Jac p = g1_load(gens + i);
        if (g1_is_identity(p)) continue;
        const G1Jac zzp = g1_mul_abs_z(g1_mul_abs_z(p));
        G1Jac e = p;
        e.x = fq_mul(e.x, fq_beta_mont());
        const G1Jac lhs = g1_add_call(e, p);
        if (!g1_is_identity(g1_add_call(zzp, g1_neg(lhs)))) atomicOr(bad, 1u);
    }
}

// *ok = every generator has order dividing r.  One small device-to-host copy per call for the fingerprint;
// the check itself runs once per distinct set.
static int generators_have_order_r(const G1Jac* d_gens, size_t n, bool* ok, Scratch& scratch, cudaStream_t s) {
    static std::mutex mu;
    static std::map<unsigned long long, bool> verdicts;
    const size_t head = n < 4 ? n : 4, tail = n < 8 ? n - head : 4;
    unsigned char sample[8 * sizeof(G1Jac)];
    ZKB_CUDA(cudaMemcpyAsync(sample, d_gens, head * sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
    if (tail) ZKB_CUDA(cudaMemcpyAsync(sample + head * sizeof(G1Jac), d_gens + (n - tail), tail * sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    unsigned long long key = 0xcbf29ce484222325ull ^ (unsigned long long)n;
    for (size_t i = 0; i < (head + tail) * sizeof(G1Jac); ++i) key = (key ^ sample[i]) * 0x100000001b3ull;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto it = verdicts.find(key);
        if (it != verdicts.end()) { *ok = it->second; return ZKB_OK; }
    }
    unsigned* d_bad = scratch.get_n<unsigned>(4);
    if (!d_bad) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemsetAsync(d_bad, 0, 16, s));
    ZKB_LAUNCH(g1_order_check_kernel, grid_for(n, 128), 128, 0, s, d_gens, n, d_bad);
    unsigned h_bad = 0;
    ZKB_CUDA(cudaMemcpyAsync(&h_bad, d_bad, 4, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    *ok = h_bad == 0;
    std::lock_guard<std::mutex> lk(mu);
    if (verdicts.size() > 4096) verdicts.clear();
    verdicts[key] = *ok;
    return ZKB_OK;
}

// The fold of me_open_step for any curve points: g' = g_odd + [u] (g_even - g_odd), u read as 256 raw bits.
__global__ void __launch_bounds__(128) me_open_fold_generic_kernel(const G1Aff* __restrict__ bases, size_t old_size, size_t new_size,
                                                                    Fr u_raw, G1Jac* __restrict__ ngen) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < new_size; g += (size_t)gridDim.x * blockDim.x) {
        const G1Aff a0 = g1_aff_load(bases + 2 * g);
        if (2 * g + 1 >= old_size) {
            g1_store(ngen + g, g1_mul_bits(g1_from_aff(a0), u_raw));
            continue;
        }
        const G1Aff a1 = g1_aff_load(bases + 2 * g + 1);
        const G1Jac diff = g1_add_mixed(g1_from_aff(a0), g1_aff_neg(a1));
        g1_store(ngen + g, g1_add_mixed(g1_mul_bits(diff, u_raw), a1));
    }
}

// ---- the last rounds of an opening, all at once --------------------------------
// Once a round has at most kTailLen generators g (affine, in the order-r group),
// every later generator is a known combination of them: with
//   g'[j] = u g[2j] + (1-u) g[2j+1]
// the generators t rounds on are g_t[j] = sum_b W_t(b) g[j 2^t + b], where
//   W_0 = [1],  W_t+1(b) = u_t W_t(b) for b < 2^t,  (1-u_t) W_t(b - 2^t) above.
// So T, T0, T1 of all remaining rounds, and the final generator, are rows of one
// MSM over g: no generator is folded any more and the chain of short, latency-bound
// rounds becomes a single call.
static constexpr size_t kTailLen = 4096;

// One block.  S[t*c + j]: scalars after t folds (t = 0..K);  Wt[t*c + b]: W_t(b) in
// Montgomery form for b < min(2^t, c).
__global__ void __launch_bounds__(1024) me_open_tail_prep_kernel(const Fr* __restrict__ s0, size_t c, const Fr* __restrict__ u_mont,
                                                                  unsigned K, Fr* __restrict__ S, Fr* __restrict__ Wt) {
    const Fr one = fe_mont_one<FrP>();
    for (size_t i = threadIdx.x; i < c; i += blockDim.x) fr_store(S + i, fr_load(s0 + i));
    if (threadIdx.x == 0) fr_store(Wt, one);
    __syncthreads();
    size_t len = c, wl = 1;
    for (unsigned t = 0; t < K; ++t) {
        const Fr u = fr_load(u_mont + t);
        const Fr v = fr_sub(one, u);
        const size_t nl = (len + 1) / 2;
        const size_t nw = 2 * wl < c ? 2 * wl : c;
        const Fr* St = S + (size_t)t * c;
        const Fr* Wc = Wt + (size_t)t * c;
        for (size_t j = threadIdx.x; j < nl; j += blockDim.x) {
            const Fr a = fr_load(St + 2 * j);
            const Fr b = 2 * j + 1 < len ? fr_load(St + 2 * j + 1) : fr_zero();
            fr_store(S + (size_t)(t + 1) * c + j, fr_add(a, fr_mmul(u, fr_sub(b, a))));
        }
        for (size_t b = threadIdx.x; b < nw; b += blockDim.x)
            fr_store(Wt + (size_t)(t + 1) * c + b, b < wl ? fr_mmul(u, fr_load(Wc + b)) : fr_mmul(v, fr_load(Wc + b - wl)));
        __syncthreads();
        len = nl;
        wl = nw;
    }
}

// rows[q*c + i], q = 3t + {0: T, 1: T0, 2: T1} of tail round t, q = 3K: the final
// generator.  A scalar's raw limbs times W, as plain integer limbs.
__global__ void me_open_tail_rows_kernel(const Fr* __restrict__ S, const Fr* __restrict__ Wt, size_t c, unsigned K,
                                         Fr* __restrict__ rows) {
    const size_t total = (3 * (size_t)K + 1) * c;
    for (size_t x = blockIdx.x * (size_t)blockDim.x + threadIdx.x; x < total; x += (size_t)gridDim.x * blockDim.x) {
        const size_t q = x / c, i = x % c;
        const unsigned t = (unsigned)(q / 3), kind = (unsigned)(q % 3);
        if (q == 3 * (size_t)K) {
            Fr one_std = fr_zero();
            one_std.v[0] = 1;
            // g_K[0] takes the first 2^K generators only
            const bool inside = K >= 63 || i < ((size_t)1 << K);
            fr_store(rows + x, inside ? fr_mmul(fr_load(Wt + (size_t)K * c + i), one_std) : fr_zero());
            continue;
        }
        const size_t j = t < 63 ? i >> t : 0;
        const size_t b = t < 63 ? i & (((size_t)1 << t) - 1) : i;
        const size_t len = t < 63 ? (c + (((size_t)1 << t) - 1)) >> t : 1;
        const Fr* St = S + (size_t)t * c;
        Fr sc = fr_zero();
        bool live = true;
        if (kind == 0) sc = fr_load(St + j);
        else if (kind == 1) { if (j & 1) sc = fr_load(St + j - 1); else live = false; }
        else { if (!(j & 1) && j + 1 < len) sc = fr_load(St + j + 1); else live = false; }
        fr_store(rows + x, live ? fr_mmul(sc, fr_load(Wt + (size_t)t * c + b)) : fr_zero());
    }
}

// out[row] = sum over the ranks p of part[p * rows + row], added in rank order
__global__ void __launch_bounds__(128) g1_sum_ranks_kernel(const G1Jac* __restrict__ part, size_t rows, unsigned world, G1Jac* __restrict__ out) {
    for (size_t row = blockIdx.x * (size_t)blockDim.x + threadIdx.x; row < rows; row += (size_t)gridDim.x * blockDim.x) {
        G1Jac acc = g1_load(part + row);
        for (unsigned p = 1; p < world; ++p) acc = g1_add_call(acc, g1_load(part + (size_t)p * rows + row));
        g1_store(out + row, acc);
    }
}

}  // namespace zkb

using namespace zkb;

extern "C" {

int zkb_commit_i32(const zkb_g1_t* d_gens, size_t n_gen, const int32_t* d_scalars, size_t n_scalars,
                   zkb_g1_t* d_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    Scratch scratch(s);
    return commit_i32_device(reinterpret_cast<const G1Jac*>(d_gens), n_gen, d_scalars, n_scalars,
                             reinterpret_cast<G1Jac*>(d_out), scratch, s);
}

int zkb_commit_i32_method(const zkb_g1_t* d_gens, size_t n_gen, const int32_t* d_scalars, size_t n_scalars,
                          zkb_g1_t* d_out, int method, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    Scratch scratch(s);
    return commit_i32_device(reinterpret_cast<const G1Jac*>(d_gens), n_gen, d_scalars, n_scalars,
                             reinterpret_cast<G1Jac*>(d_out), scratch, s, method);
}

// Rows [begin, end) of rank `rank` when m rows are dealt out in contiguous blocks; the first m % world ranks take one more.
static void row_block(size_t m, int world, int rank, size_t* begin, size_t* end) {
    const size_t base = m / world, extra = m % world;
    *begin = (size_t)rank * base + ((size_t)rank < extra ? (size_t)rank : extra);
    *end = *begin + base + ((size_t)rank < extra ? 1 : 0);
}

int zkb_commit_i32_sharded(const zkb_g1_t* d_gens, size_t n_gen, const int32_t* d_scalars_local, size_t rows_local,
                           size_t rows_total, zkb_g1_t* d_out_all, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    const int world = comm_world(), rank = comm_rank();
    if (world < 1) return fail(ZKB_ERR_ARG, "comm: not initialised (zkb_comm_init)");
    if (n_gen == 0) return fail(ZKB_ERR_DIM, "Commitment::commit_int - Incompatible dimensions");
    size_t begin, end;
    row_block(rows_total, world, rank, &begin, &end);
    if (rows_local != end - begin) return fail(ZKB_ERR_DIM, "commit: this rank's row count does not match its block of the rows");
    if (rows_total == 0) return ZKB_OK;
    G1Jac* out = reinterpret_cast<G1Jac*>(d_out_all);
    Scratch scratch(s);
    if (rows_total % world == 0) {
        // equal blocks: every rank commits into its slot of the result and the gather runs in place
        if (rows_local)
            ZKB_TRY(commit_i32_device(reinterpret_cast<const G1Jac*>(d_gens), n_gen, d_scalars_local, rows_local * n_gen,
                                      out + begin, scratch, s));
        return comm_allgather(out + begin, out, rows_local * sizeof(G1Jac), s);
    }
    const size_t max_rows = (rows_total + world - 1) / world;
    G1Jac* send = scratch.get_n<G1Jac>(max_rows);
    G1Jac* recv = scratch.get_n<G1Jac>(max_rows * world);
    if (!send || !recv) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemsetAsync(send, 0, max_rows * sizeof(G1Jac), s));
    if (rows_local)
        ZKB_TRY(commit_i32_device(reinterpret_cast<const G1Jac*>(d_gens), n_gen, d_scalars_local, rows_local * n_gen, send, scratch, s));
    ZKB_TRY(comm_allgather(send, recv, max_rows * sizeof(G1Jac), s));
    for (int p = 0; p < world; ++p) {
        size_t b, e;
        row_block(rows_total, world, p, &b, &e);
        if (e > b) ZKB_CUDA(cudaMemcpyAsync(out + b, recv + (size_t)p * max_rows, (e - b) * sizeof(G1Jac), cudaMemcpyDeviceToDevice, s));
    }
    return ZKB_OK;
}

int zkb_commit_i32_colsharded(const zkb_g1_t* d_gens_local, size_t n_gen_local, const int32_t* d_scalars_local, size_t rows,
                              zkb_g1_t* d_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    const int world = comm_world();
    if (world < 1) return fail(ZKB_ERR_ARG, "comm: not initialised (zkb_comm_init)");
    if (rows == 0) return ZKB_OK;
    if (rows > 0xffffffffull) return fail(ZKB_ERR_LIMIT, "commit: too many rows");
    Scratch scratch(s);
    G1Jac* mine = scratch.get_n<G1Jac>(rows);
    G1Jac* all = scratch.get_n<G1Jac>(rows * (size_t)world);
    if (!mine || !all) return ZKB_ERR_CUDA;
    if (n_gen_local) {
        ZKB_TRY(commit_i32_device(reinterpret_cast<const G1Jac*>(d_gens_local), n_gen_local, d_scalars_local, rows * n_gen_local, mine,
                                  scratch, s));
    } else {
        ZKB_CUDA(cudaMemsetAsync(mine, 0, rows * sizeof(G1Jac), s));      // no columns here: the identity for every row
    }
    ZKB_TRY(comm_allgather(mine, all, rows * sizeof(G1Jac), s));
    ZKB_LAUNCH(g1_sum_ranks_kernel, grid_for(rows, 128), 128, 0, s, all, rows, (unsigned)world, reinterpret_cast<G1Jac*>(d_out));
    return ZKB_OK;
}

int zkb_commit_int(const zkb_g1_t* d_gens, size_t n_gen, const zkb_fr_t* d_scalars, size_t n_scalars,
                   zkb_g1_t* d_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (n_gen == 0 || n_scalars % n_gen) return fail(ZKB_ERR_DIM, "Commitment::commit_int - Incompatible dimensions");
    if (n_scalars == 0) return ZKB_OK;
    Scratch scratch(s);
    int32_t* ints = scratch.get_n<int32_t>(n_scalars);
    if (!ints) return ZKB_ERR_CUDA;
    ZKB_TRY(zkb_fr_to_i32(d_scalars, ints, n_scalars, stream));
    return commit_i32_device(reinterpret_cast<const G1Jac*>(d_gens), n_gen, ints, n_scalars,
                             reinterpret_cast<G1Jac*>(d_out), scratch, s);
}

int zkb_commit_i32_host(const zkb_g1_t* h_gens, size_t n_gen, const int32_t* h_scalars, size_t n_scalars,
                        zkb_g1_t* h_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (n_gen == 0 || n_scalars % n_gen) return fail(ZKB_ERR_DIM, "Commitment::commit_int - Incompatible dimensions");
    const size_t m = n_scalars / n_gen;
    if (m == 0) return ZKB_OK;
    Scratch scratch(s);
    G1Jac* d_gens = scratch.get_n<G1Jac>(n_gen);
    int32_t* d_sc = scratch.get_n<int32_t>(n_scalars);
    G1Jac* d_out = scratch.get_n<G1Jac>(m);
    if (!d_gens || !d_sc || !d_out) return ZKB_ERR_CUDA;
    ZKB_CUDA(cudaMemcpyAsync(d_gens, h_gens, n_gen * sizeof(G1Jac), cudaMemcpyHostToDevice, s));
    // The combination tables depend on the generators only.  When the shape makes them the likely choice (decided
    // for 16-bit scalars; the real choice follows once the scalars are here and their range is known), they are
    // built on the caller's stream while the scalars cross the bus on the second stream.
    const G1Aff* early_table = nullptr;
    SideStream* side = nullptr;
    const int w3_guess = comb_windows_for_max(1u << 15), w7_guess = windows_for_max(1u << 15);
    if (m >= 64 && comb_table_bytes(n_gen) <= kCombTableLimit && comb_cost(m, n_gen, w3_guess) < bucket_cost(m, n_gen, w7_guess))
        side = side_stream();
    if (side) {
        std::lock_guard<std::mutex> turn(side->busy);
        Drain drain{side->st};
        ZKB_CUDA(cudaEventRecord(side->fork, s));                 // d_sc exists from here on in s's order
        ZKB_CUDA(cudaStreamWaitEvent(side->st, side->fork, 0));
        ZKB_CUDA(cudaMemcpyAsync(d_sc, h_scalars, n_scalars * sizeof(int32_t), cudaMemcpyHostToDevice, side->st));
        ZKB_CUDA(cudaEventRecord(side->join, side->st));
        G1Aff* bases = scratch.get_n<G1Aff>(n_gen);
        if (!bases) return ZKB_ERR_CUDA;
        ZKB_TRY(to_affine_device(d_gens, bases, n_gen, s));
        ZKB_TRY(comb_tables_build(bases, n_gen, &early_table, scratch, s));
        ZKB_CUDA(cudaStreamWaitEvent(s, side->join, 0));
        ZKB_TRY(commit_i32_device(d_gens, n_gen, d_sc, n_scalars, d_out, scratch, s, ZKB_MSM_AUTO, early_table));
        ZKB_CUDA(cudaMemcpyAsync(h_out, d_out, m * sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
        ZKB_CUDA(cudaStreamSynchronize(s));
        return ZKB_OK;
    }
    ZKB_CUDA(cudaMemcpyAsync(d_sc, h_scalars, n_scalars * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    ZKB_TRY(commit_i32_device(d_gens, n_gen, d_sc, n_scalars, d_out, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_out, d_out, m * sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_commit(const zkb_g1_t* d_gens, size_t n_gen, const zkb_fr_t* d_scalars, size_t n_scalars,
               zkb_g1_t* d_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (n_gen == 0 || n_scalars % n_gen) return fail(ZKB_ERR_DIM, "Commitment::commit - Incompatible dimensions");
    if (n_scalars == 0) return ZKB_OK;
    Scratch scratch(s);
    return msm_rows<true>(reinterpret_cast<const G1Jac*>(d_gens), n_gen, d_scalars, n_scalars / n_gen, kMaxWindows,
                          reinterpret_cast<G1Jac*>(d_out), scratch, s);
}

}  // extern "C"

// What has to outlive the enqueueing of an opening: host arrays the copies read, and where the results are.
struct OpenState {
    std::vector<zkb_fr_t> coef, um;
    G1Jac* d_proof = nullptr;      // 3 k + 1 proof elements
    const Fr* cs = nullptr;        // the fully folded scalar
};

// Queues one opening on `s` (generator chain) and side->st (the MSMs); on return `s` has taken the side stream's
// work back, and st says where the results will be.  Reads h_u only while it runs.
static int me_open_enqueue(const zkb_fr_t* d_t, const zkb_g1_t* d_gens, size_t n, const zkb_fr_t* h_u, unsigned k,
                           cudaStream_t s, SideStream* side, Scratch& keep, OpenState& st) {
    // The chain that cannot be shortened is generators -> affine -> folded
    // generators, round after round, on the caller's stream.  The three-row MSM of
    // a round only reads that round's affine generators and scalar rows, so it runs
    // on a second stream beside the later rounds; every round has its own slice
    // of `rows` and `bases` (the lengths halve, 2n + k entries cover them all).
    const size_t h0 = (n + 1) / 2, total = 2 * n + k + 2;
    Fr* sc[2] = {keep.get_n<Fr>(h0), keep.get_n<Fr>(h0)};
    G1Jac* gn[2] = {keep.get_n<G1Jac>(h0), keep.get_n<G1Jac>(h0)};
    Fr* rows = keep.get_n<Fr>(3 * total);
    G1Aff* bases = keep.get_n<G1Aff>(total);
    G1Jac* d_proof = keep.get_n<G1Jac>(3 * (size_t)k + 1);
    if (!sc[0] || !sc[1] || !gn[0] || !gn[1] || !rows || !bases || !d_proof) return ZKB_ERR_CUDA;
    const Fr* cs = reinterpret_cast<const Fr*>(d_t);
    const G1Jac* cg = reinterpret_cast<const G1Jac*>(d_gens);
    size_t cur = n, used = 0;
    auto host_fr = [](const zkb_fr_t& h) { Fr r; memcpy(&r, &h, sizeof(Fr)); return r; };
    int rc = ZKB_OK;
    // Rounds above kTailLen generators ("big" rounds): each one only forms its bucket
    // sums on the side stream; all share one segment count, so a single reduction
    // after the last of them turns the buckets of every round into proof points
    // (the Horner chain over 37 windows is latency-bound: once, not once per round).
    bool order_r = true;
    ZKB_TRY(generators_have_order_r(reinterpret_cast<const G1Jac*>(d_gens), n, &order_r, keep, s));
    unsigned n_big = 0;
    for (size_t c = n; n_big < k && (c > kTailLen || !order_r); c = (c + 1) / 2) ++n_big;
    // The two small host arrays of an opening (combination scalars of the derived T rows, Montgomery forms of the
    // tail's challenges) depend on h_u only.  They go to the device NOW, while both streams are still empty: a copy
    // from pageable host memory waits for the work queued before it, which later on would be most of the opening.
    std::vector<zkb_fr_t>& coef = st.coef;
    Fr* d_coef = nullptr;
    if (n_big > 1 && order_r) {
        // coefficient of every point of big_points[0 .. 2 n_big - 1) in T of round t = 1 .. n_big - 1
        const size_t n_pts = 2 * (size_t)n_big - 1, n_der = n_big - 1;
        std::vector<hfr::H> a(n_big), b(n_big), c(n_big);
        for (unsigned i = 0; i < n_big; ++i) {
            hfr::H u = hfr::load(h_u[i]);
            for (int pass = 0; pass < 2; ++pass)      // a raw value of r or more names the same multiple as its residue
                if (hfr::geq(u, hfr::kMod)) { uint64_t bo; u = hfr::raw_sub(u, hfr::kMod, &bo); }
            const hfr::H v = hfr::sub(hfr::from_u64(1), u);
            a[i] = hfr::mul(u, v);
            b[i] = hfr::mul(v, v);
            c[i] = hfr::mul(u, u);
        }
        coef.assign(n_der * n_pts, hfr::store(hfr::zero()));
        for (unsigned t = 1; t < n_big; ++t) {
            zkb_fr_t* row = &coef[(size_t)(t - 1) * n_pts];
            hfr::H run = hfr::from_u64(1);            // product of a_i for i in (j, t)
            for (int j = (int)t - 1; j >= 0; --j) {
                row[1 + 2 * (size_t)j] = hfr::store(hfr::mul(b[j], run));
                row[2 + 2 * (size_t)j] = hfr::store(hfr::mul(c[j], run));
                run = hfr::mul(run, a[j]);
            }
            row[0] = hfr::store(run);
        }
        d_coef = keep.get_n<Fr>(coef.size());
        if (!d_coef) return ZKB_ERR_CUDA;
        ZKB_CUDA(cudaMemcpyAsync(d_coef, coef.data(), coef.size() * sizeof(Fr), cudaMemcpyHostToDevice, s));
    }
    std::vector<zkb_fr_t>& um = st.um;
    Fr* d_um = nullptr;
    if (k > n_big) {
        um.assign(k - n_big, zkb_fr_t());
        for (unsigned t = 0; t < k - n_big; ++t) um[t] = hfr::store(hfr::to_mont(hfr::load(h_u[n_big + t])));
        d_um = keep.get_n<Fr>(k - n_big);
        if (!d_um) return ZKB_ERR_CUDA;
        ZKB_CUDA(cudaMemcpyAsync(d_um, um.data(), (k - n_big) * sizeof(Fr), cudaMemcpyHostToDevice, s));
    }
    // Only the first big round forms T = sum s_i g_i by an MSM.  With a = u (1 - u), b = (1 - u)^2, c = u^2 of a
    // round, the next round's T is  a T + b T0 + c T1  (expand sum s'_j g'_j with the two folds above), so
    // every later T is a fixed combination of the first T and the T0, T1 of the rounds before it: rounds
    // after the first need two MSM rows instead of three, and all derived T come from one small MSM over
    // those proof points at the end.  Like the fold and the tail this uses scalars modulo r.
    MsmShape big0;
    G1Jac* big_buckets = nullptr;
    G1Jac* big_points = nullptr;                 // T, T0, T1 of round 0, then T0, T1 of every later big round
    size_t per_row = 0;
    const size_t big_rows = !n_big ? 0 : (order_r ? 3 + 2 * (size_t)(n_big - 1) : 3 * (size_t)n_big);
    if (n_big) {
        if (order_r) ZKB_TRY(msm_shape(2 * n, 3, kGlvWindows, true, 0, &big0));
        else ZKB_TRY(msm_shape(n, 3, kMaxWindows, true, 0, &big0));
        per_row = msm_bucket_count(big0) / 3;
        big_buckets = keep.get_n<G1Jac>(per_row * big_rows);
        big_points = keep.get_n<G1Jac>(big_rows);
        if (!big_buckets || !big_points) return ZKB_ERR_CUDA;
    }
    unsigned r = 0;
    size_t rows_done = 0;
    for (; r < n_big && rc == ZKB_OK; ++r) {
        const size_t nn = (cur + 1) / 2;
        const unsigned n_rows = (r == 0 || !order_r) ? 3u : 2u;
        const Fr u_mont = host_fr(hfr::store(hfr::to_mont(hfr::load(h_u[r]))));
        Fr* rows_r = rows + 3 * used;
        G1Aff* bases_r = bases + used;
        ZKB_LAUNCH(me_open_rows_kernel, grid_for(nn, 128), 128, 0, s, cs, cur, nn, u_mont, n_rows == 3 ? 1u : 0u, rows_r, sc[r & 1]);
        ZKB_TRY(to_affine_device(cg, bases_r, cur, s));
        ZKB_CUDA(cudaEventRecord(side->fork, s));
        ZKB_CUDA(cudaStreamWaitEvent(side->st, side->fork, 0));
        {
            Scratch round(side->st);   // sorted lists of this round, released in the side stream's order
            MsmShape sh;
            if (order_r) {
                G1Aff* b2 = nullptr;
                Fr* r2 = nullptr;
                rc = glv_expand(bases_r, cur, rows_r, n_rows, &b2, &r2, round, side->st);
                if (rc == ZKB_OK) rc = msm_shape(2 * cur, n_rows, kGlvWindows, true, big0.nseg, &sh);
                if (rc == ZKB_OK) rc = msm_accumulate_phase<true>(b2, r2, sh, big_buckets + per_row * rows_done, round, side->st);
            } else {
                rc = msm_shape(cur, n_rows, kMaxWindows, true, big0.nseg, &sh);
                if (rc == ZKB_OK) rc = msm_accumulate_phase<true>(bases_r, rows_r, sh, big_buckets + per_row * rows_done, round, side->st);
            }
        }
        if (order_r) {
            ZKB_LAUNCH(me_open_fold_kernel, grid_for(nn, ZKB_FOLD_THREADS), ZKB_FOLD_THREADS, 0, s, bases_r, cur, nn, fold_digits(h_u[r]), gn[r & 1]);
        } else {
            ZKB_LAUNCH(me_open_fold_generic_kernel, grid_for(nn, 128), 128, 0, s, bases_r, cur, nn, host_fr(h_u[r]), gn[r & 1]);
        }
        cs = sc[r & 1];
        cg = gn[r & 1];
        used += cur;
        cur = nn;
        rows_done += n_rows;
    }
    if (rc == ZKB_OK && n_big) {
        MsmShape all = big0;
        all.m = big_rows;
        Scratch fin(side->st);
        rc = msm_reduce_phase(big_buckets, all, big_points, fin, side->st);
        if (rc == ZKB_OK && !order_r)      // three rows per round, already in proof order
            ZKB_CUDA(cudaMemcpyAsync(d_proof, big_points, big_rows * sizeof(G1Jac), cudaMemcpyDeviceToDevice, side->st));
        if (rc == ZKB_OK && order_r) ZKB_CUDA(cudaMemcpyAsync(d_proof, big_points, 3 * sizeof(G1Jac), cudaMemcpyDeviceToDevice, side->st));
        for (unsigned t = 1; t < n_big && rc == ZKB_OK && order_r; ++t)
            ZKB_CUDA(cudaMemcpyAsync(d_proof + 3 * (size_t)t + 1, big_points + 3 + 2 * (size_t)(t - 1), 2 * sizeof(G1Jac),
                                     cudaMemcpyDeviceToDevice, side->st));
        if (rc == ZKB_OK && n_big > 1 && order_r) {
            // the derived T rows: one small MSM over the proof points so far, with the scalars copied at the start
            const size_t n_pts = 2 * (size_t)n_big - 1, n_der = n_big - 1;
            G1Jac* d_der = fin.get_n<G1Jac>(n_der);
            if (!d_der) return ZKB_ERR_CUDA;
            G1Aff* pts_aff = fin.get_n<G1Aff>(n_pts);
            if (!pts_aff) return ZKB_ERR_CUDA;
            rc = to_affine_device(big_points, pts_aff, n_pts, side->st);
            if (rc == ZKB_OK) rc = msm_rows_affine_glv(pts_aff, n_pts, d_coef, n_der, d_der, fin, side->st);
            for (unsigned t = 1; t < n_big && rc == ZKB_OK; ++t)
                ZKB_CUDA(cudaMemcpyAsync(d_proof + 3 * (size_t)t, d_der + (t - 1), sizeof(G1Jac), cudaMemcpyDeviceToDevice, side->st));
        }
    }
    // the remaining K rounds and the final generator as one MSM over this round's generators
    const unsigned K = k - r;
    if (rc == ZKB_OK && K > 0) {
        Fr* S = keep.get_n<Fr>(((size_t)K + 1) * cur);
        Fr* Wt = keep.get_n<Fr>(((size_t)K + 1) * cur);
        Fr* tail_rows = keep.get_n<Fr>((3 * (size_t)K + 1) * cur);
        G1Aff* bases_t = bases + used;
        if (!d_um || !S || !Wt || !tail_rows) return ZKB_ERR_CUDA;
        ZKB_LAUNCH(me_open_tail_prep_kernel, 1, 1024, 0, s, cs, cur, d_um, K, S, Wt);
        ZKB_LAUNCH(me_open_tail_rows_kernel, grid_for((3 * (size_t)K + 1) * cur, 128), 128, 0, s, S, Wt, cur, K, tail_rows);
        ZKB_TRY(to_affine_device(cg, bases_t, cur, s));
        rc = msm_rows_affine_glv(bases_t, cur, tail_rows, 3 * (size_t)K + 1, d_proof + 3 * r, keep, s);
        cs = S + (size_t)K * cur;   // the fully folded scalar
    }
    // the caller's stream takes the side stream's work back before anything is read or released
    ZKB_CUDA(cudaEventRecord(side->join, side->st));
    ZKB_CUDA(cudaStreamWaitEvent(s, side->join, 0));
    if (rc != ZKB_OK) return rc;
    if (K == 0) ZKB_CUDA(cudaMemcpyAsync(d_proof + 3 * k, cg, sizeof(G1Jac), cudaMemcpyDeviceToDevice, s));
    st.d_proof = d_proof;
    st.cs = cs;
    return ZKB_OK;
}

// ---- openings in flight: zkb_me_open_begin / zkb_me_open_end -------------------------------
// An opening is bound by the multiplier, a lookup proof by memory, and an opening's small rounds by latency: a caller
// that starts an opening, goes on with other proofs and collects the result later overlaps all three.  Each opening in
// flight has its own pair of non-blocking streams (a lane), its scratch memory bound to that lane, and a page-locked
// block for the results; at most kOpenLanes per device, a further begin runs the opening at once instead.
static constexpr int kOpenLanes = 4;
struct OpenLane {
    bool made = false, busy = false;
    cudaStream_t a = nullptr;
    SideStream side;
    cudaEvent_t ready = nullptr;
    char* pinned = nullptr;        // (3 * 62 + 1) proof elements and the opening
};
static constexpr size_t kOpenPinned = (3 * 62 + 1) * sizeof(G1Jac) + 32;
struct OpenJob {
    OpenLane* lane = nullptr;      // nullptr: the opening ran inside begin, results are in `done_*`
    Scratch keep;
    OpenState st;
    unsigned k = 0;
    std::vector<zkb_g1_t> done_proof;
    zkb_fr_t done_out;
    explicit OpenJob(cudaStream_t s) : keep(s) {}
};
static std::mutex g_lane_mu;
static OpenLane g_lanes[64][kOpenLanes];

static OpenLane* take_lane() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_lane_mu);
    for (int i = 0; i < kOpenLanes; ++i) {
        OpenLane& l = g_lanes[dev][i];
        if (l.busy) continue;
        if (!l.made) {
            void* p = nullptr;
            if (cudaStreamCreateWithFlags(&l.a, cudaStreamNonBlocking) != cudaSuccess ||
                cudaStreamCreateWithFlags(&l.side.st, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&l.side.fork, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&l.side.join, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&l.ready, cudaEventDisableTiming) != cudaSuccess ||
                cudaHostAlloc(&p, kOpenPinned, cudaHostAllocDefault) != cudaSuccess) {
                cudaGetLastError();
                return nullptr;
            }
            l.pinned = static_cast<char*>(p);
            l.made = true;
        }
        l.busy = true;
        return &l;
    }
    return nullptr;
}
static void release_lane(OpenLane* l) {
    std::lock_guard<std::mutex> lk(g_lane_mu);
    l->busy = false;
}

extern "C" {

int zkb_me_open(const zkb_fr_t* d_t, const zkb_g1_t* d_gens, size_t n, const zkb_fr_t* h_u, unsigned k,
                zkb_g1_t* h_proof, zkb_fr_t* h_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (n == 0) return fail(ZKB_ERR_DIM, "Commitment::me_open - Incompatible dimensions");
    if (k > 62) return fail(ZKB_ERR_LIMIT, "Commitment::me_open - more than 62 rounds");
    SideStream* side = side_stream();
    if (!side) return ZKB_ERR_CUDA;
    std::lock_guard<std::mutex> turn(side->busy);
    Scratch keep(s);
    Drain drain{side->st};   // destroyed before `keep`: nothing of the side stream outlives the buffers
    OpenState st;
    const int rc = me_open_enqueue(d_t, d_gens, n, h_u, k, s, side, keep, st);
    if (rc != ZKB_OK) {
        cudaStreamSynchronize(s);
        return rc;
    }
    ZKB_CUDA(cudaMemcpyAsync(h_proof, st.d_proof, (3 * (size_t)k + 1) * sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaMemcpyAsync(h_out, st.cs, 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_me_open_begin(const zkb_fr_t* d_t, const zkb_g1_t* d_gens, size_t n, const zkb_fr_t* h_u, unsigned k, void* stream,
                      void** handle) {
    ZKB_API_RANGE();
    if (!handle) return fail(ZKB_ERR_ARG, "me_open_begin: null handle");
    *handle = nullptr;
    if (n == 0) return fail(ZKB_ERR_DIM, "Commitment::me_open - Incompatible dimensions");
    if (k > 62) return fail(ZKB_ERR_LIMIT, "Commitment::me_open - more than 62 rounds");
    OpenLane* lane = take_lane();
    if (!lane) {                    // every lane is in use: the opening runs now
        OpenJob* job = new OpenJob(as_stream(stream));
        job->k = k;
        job->done_proof.resize(3 * (size_t)k + 1);
        const int rc = zkb_me_open(d_t, d_gens, n, h_u, k, job->done_proof.data(), &job->done_out, stream);
        if (rc != ZKB_OK) { delete job; return rc; }
        *handle = job;
        return ZKB_OK;
    }
    OpenJob* job = new OpenJob(lane->a);
    job->lane = lane;
    job->k = k;
    int rc = ZKB_OK;
    if (cudaEventRecord(lane->ready, as_stream(stream)) != cudaSuccess || cudaStreamWaitEvent(lane->a, lane->ready, 0) != cudaSuccess)
        rc = fail(ZKB_ERR_CUDA, "me_open_begin: cannot order the opening after the caller's stream");
    if (rc == ZKB_OK) rc = me_open_enqueue(d_t, d_gens, n, h_u, k, lane->a, &lane->side, job->keep, job->st);
    if (rc == ZKB_OK) {
        const size_t pb = (3 * (size_t)k + 1) * sizeof(G1Jac);
        if (cudaMemcpyAsync(lane->pinned, job->st.d_proof, pb, cudaMemcpyDeviceToHost, lane->a) != cudaSuccess ||
            cudaMemcpyAsync(lane->pinned + pb, job->st.cs, 32, cudaMemcpyDeviceToHost, lane->a) != cudaSuccess)
            rc = fail(ZKB_ERR_CUDA, "me_open_begin: cannot queue the result copies");
    }
    if (rc != ZKB_OK) {
        cudaStreamSynchronize(lane->side.st);
        cudaStreamSynchronize(lane->a);
        delete job;
        release_lane(lane);
        return rc;
    }
    *handle = job;
    return ZKB_OK;
}

int zkb_me_open_end(void* handle, zkb_g1_t* h_proof, zkb_fr_t* h_out) {
    if (!handle) return fail(ZKB_ERR_ARG, "me_open_end: null handle");
    OpenJob* job = static_cast<OpenJob*>(handle);
    const size_t pb = (3 * (size_t)job->k + 1) * sizeof(G1Jac);
    int rc = ZKB_OK;
    if (!job->lane) {
        if (h_proof) memcpy(h_proof, job->done_proof.data(), pb);
        if (h_out) *h_out = job->done_out;
    } else {
        const cudaError_t e1 = cudaStreamSynchronize(job->lane->a), e2 = cudaStreamSynchronize(job->lane->side.st);
        if (e1 != cudaSuccess || e2 != cudaSuccess) rc = cuda_fail(e1 != cudaSuccess ? e1 : e2, "me_open_end");
        else {
            if (h_proof) memcpy(h_proof, job->lane->pinned, pb);
            if (h_out) memcpy(h_out, job->lane->pinned + pb, 32);
        }
    }
    OpenLane* lane = job->lane;
    delete job;                      // the scratch memory goes back in the lane's stream order
    if (lane) release_lane(lane);
    return rc;
}

}  // extern "C"
