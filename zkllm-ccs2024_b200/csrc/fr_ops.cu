// FrTensor device work: conversions, elementwise field ops, sums, multilinear
// folds expressed as dot products with eq-tables, layout utilities, matmul.
//
// All tensors hold standard-form values.  Products against a challenge use the
// challenge in Montgomery form (montmul(x, u*R) = x*u), products of two tensor
// values are corrected by one multiplication with R^2 per output.
#include "frutil.cuh"
#include "hostfr.hpp"

#include <vector>

namespace zkb {

static constexpr unsigned kThreads = 256;

// ---------------------------------------------------------------------------
// elementwise
// ---------------------------------------------------------------------------
enum class BinOp { Add, Sub, Mul, MontMul };
enum class UnOp { Neg, Mont, Unmont };

template <BinOp OP>
__global__ void __launch_bounds__(kThreads) fr_binary_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b,
                                                              Fr* __restrict__ out, size_t n) {
    const Fr r2 = fe_r2<FrP>();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        Fr x = fr_load(a + i), y = fr_load(b + i), z;
        if (OP == BinOp::Add) z = fr_add(x, y);
        else if (OP == BinOp::Sub) z = fr_sub(x, y);
        else if (OP == BinOp::Mul) z = fr_mmul(fr_mmul(x, y), r2);
        else z = fr_mmul(x, y);
        fr_store(out + i, z);
    }
}

// y is the broadcast operand; for Mul it arrives already in Montgomery form
template <BinOp OP>
__global__ void __launch_bounds__(kThreads) fr_scalar_kernel(const Fr* __restrict__ a, Fr y, Fr* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        Fr x = fr_load(a + i), z;
        if (OP == BinOp::Add) z = fr_add(x, y);
        else if (OP == BinOp::Sub) z = fr_sub(x, y);
        else z = fr_mmul(x, y);
        fr_store(out + i, z);
    }
}

template <UnOp OP>
__global__ void __launch_bounds__(kThreads) fr_unary_kernel(const Fr* __restrict__ a, Fr* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        Fr x = fr_load(a + i), z;
        if (OP == UnOp::Neg) z = fr_neg(x);
        else if (OP == UnOp::Mont) z = to_mont<FrP>(x);
        else z = from_mont<FrP>(x);
        fr_store(out + i, z);
    }
}

// ---------------------------------------------------------------------------
// conversions
// ---------------------------------------------------------------------------
__global__ void fr_from_i32_kernel(const int32_t* __restrict__ in, Fr* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        fr_store(out + i, fr_from_i64((long long)in[i]));
}
__global__ void fr_from_i64_kernel(const int64_t* __restrict__ in, Fr* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        fr_store(out + i, fr_from_i64((long long)in[i]));
}
__global__ void fr_to_i32_kernel(const Fr* __restrict__ in, int32_t* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = fr_to_i32(fr_load(in + i));
}
__global__ void fr_to_i64_kernel(const Fr* __restrict__ in, int64_t* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = fr_to_i64(fr_load(in + i));
}
// float_to_scalar / double_to_scalar (fr-tensor.cu:749-768): scale in the input's
// own precision, add +-0.5 in double precision, truncate toward zero.
__global__ void fr_from_f32_kernel(const float* __restrict__ in, unsigned long scale, Fr* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float x = in[i] * scale;
        long v = (x >= 0) ? static_cast<long>(x + 0.5) : static_cast<long>(x - 0.5);
        fr_store(out + i, fr_from_i64(v));
    }
}
__global__ void fr_from_f64_kernel(const double* __restrict__ in, unsigned long scale, Fr* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        double x = in[i] * scale;
        long v = (x >= 0) ? static_cast<long>(x + 0.5) : static_cast<long>(x - 0.5);
        fr_store(out + i, fr_from_i64(v));
    }
}

// ---------------------------------------------------------------------------
// sums
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) fr_partial_sum_kernel(const Fr* __restrict__ a, size_t n, Fr* __restrict__ partial) {
    __shared__ Fr red[32];
    Fr acc = fr_zero();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        acc = fr_add(acc, fr_load(a + i));
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) fr_store(partial + blockIdx.x, acc);
}
__global__ void __launch_bounds__(kThreads) fr_final_sum_kernel(const Fr* __restrict__ a, size_t n, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    Fr acc = fr_zero();
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) acc = fr_add(acc, fr_load(a + i));
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) fr_store(out, acc);
}

int launch_final_sum(const Fr* d_in, size_t n, Fr* d_out, cudaStream_t stream) {
    ZKB_LAUNCH(fr_final_sum_kernel, 1, kThreads, 0, stream, d_in, n, d_out);
    return ZKB_OK;
}

// ---------------------------------------------------------------------------
// eq tables
// ---------------------------------------------------------------------------
__global__ void eq_table_kernel(Challenges ch, unsigned k, Fr* __restrict__ table) {
    __shared__ Fr f1[32], f0[32];   // u_j * R and (1 - u_j) * R
    if (threadIdx.x < k) {
        Fr um = to_mont<FrP>(ch.u[threadIdx.x]);
        f1[threadIdx.x] = um;
        f0[threadIdx.x] = fr_sub(fe_mont_one<FrP>(), um);
    }
    __syncthreads();
    const size_t n = (size_t)1 << k;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        Fr acc = fe_mont_one<FrP>();
        for (unsigned j = 0; j < k; ++j) acc = fr_mmul(acc, ((i >> j) & 1) ? f1[j] : f0[j]);
        fr_store(table + i, acc);
    }
}

int build_eq_table(const zkb_fr_t* h_u, unsigned k, Fr* d_table, cudaStream_t stream) {
    if (k > 32) return fail(ZKB_ERR_LIMIT, "eq table: more than 32 variables");
    Challenges ch;
    memset(&ch, 0, sizeof(ch));
    for (unsigned j = 0; j < k; ++j) memcpy(ch.u[j].v, h_u[j].val, 32);
    const size_t n = (size_t)1 << k;
    ZKB_LAUNCH(eq_table_kernel, grid_for(n, kThreads), kThreads, 0, stream, ch, k, d_table);
    return ZKB_OK;
}

// ---------------------------------------------------------------------------
// dot products with eq tables
// ---------------------------------------------------------------------------
// out[o*window + w] = sum_{j<J} a[(o*J + j)*window + w] * E[j]    (E in Montgomery form)
// window == 1: one block per output row, threads stride over j.
__global__ void __launch_bounds__(kThreads) fr_rowdot_kernel(const Fr* __restrict__ a, const Fr* __restrict__ E,
                                                              size_t rows, size_t J, Fr* __restrict__ out) {
    __shared__ Fr red[32];
    for (size_t o = blockIdx.x; o < rows; o += gridDim.x) {
        const Fr* row = a + o * J;
        LazyDot dot;
        dot.init();
        for (size_t j = threadIdx.x; j < J; j += blockDim.x) dot.add(fr_load(row + j), fr_load(E + j));
        Fr acc = block_sum(dot.finish(), red);
        if (threadIdx.x == 0) fr_store(out + o, acc);
    }
}
// The same with one warp per (row, part of the j range): no block barrier, ZKB_ROWDOT_UNROLL
// loads in flight per lane.  out[p * rows + o] = partial sum of part p (parts > 1:
// the caller adds the slices).
#ifndef ZKB_ROWDOT_UNROLL
#define ZKB_ROWDOT_UNROLL 4
#endif
// Measured on W 4096 x 4096: unroll 4 with 3 CTAs per SM (80 registers) 137 us, unroll 4 with 2 CTAs (98 registers) 147 us,
// unroll 8 (130 registers, one CTA) 208 us.
#ifndef ZKB_ROWDOT_MINBLOCKS
#define ZKB_ROWDOT_MINBLOCKS 3
#endif
__global__ void __launch_bounds__(kThreads, ZKB_ROWDOT_MINBLOCKS) fr_rowdot_warp_kernel(const Fr* __restrict__ a, const Fr* __restrict__ E,
                                                                   size_t rows, size_t J, unsigned parts, Fr* __restrict__ out) {
    constexpr int U = ZKB_ROWDOT_UNROLL;
    const unsigned lane = threadIdx.x & 31u;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t jper = (J + parts - 1) / parts;
    for (size_t unit = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; unit < rows * parts; unit += warps) {
        const size_t o = unit / parts, p = unit % parts;
        const Fr* row = a + o * J;
        const size_t j0 = p * jper, j1 = (j0 + jper < J) ? j0 + jper : J;
        LazyDot dot;
        dot.init();
        size_t j = j0 + lane;
        for (; j + 32 * (U - 1) < j1; j += 32 * U) {
            Fr x[U];
#pragma unroll
            for (int t = 0; t < U; ++t) x[t] = fr_load(row + j + 32 * t);
#pragma unroll
            for (int t = 0; t < U; ++t) dot.add(x[t], fr_load(E + j + 32 * t));
        }
        for (; j < j1; j += 32) dot.add(fr_load(row + j), fr_load(E + j));
        const Fr acc = warp_sum(dot.finish());
        if (lane == 0) fr_store(out + p * rows + o, acc);
    }
}
// window > 1: one thread per output element, loop over j (coalesced across w).
// gridDim.y splits the j range; partial results go to out + blockIdx.y * (other*window).
__global__ void __launch_bounds__(kThreads) fr_coldot_kernel(const Fr* __restrict__ a, const Fr* __restrict__ E,
                                                              size_t other, size_t J, size_t window,
                                                              size_t a_len, Fr* __restrict__ out) {
    const size_t total = other * window;
    const size_t jper = (J + gridDim.y - 1) / gridDim.y;
    const size_t j0 = blockIdx.y * jper;
    const size_t j1 = (j0 + jper < J) ? j0 + jper : J;
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < total; g += (size_t)gridDim.x * blockDim.x) {
        const size_t o = g / window, w = g % window;
        LazyDot dot;
        dot.init();
        for (size_t j = j0; j < j1; ++j) {
            const size_t idx = (o * J + j) * window + w;
            if (idx < a_len) dot.add(fr_load(a + idx), fr_load(E + j));
        }
        fr_store(out + blockIdx.y * total + g, dot.finish());
    }
}
// out[g] = sum_{s<S} part[s*total + g]
__global__ void fr_sum_slices_kernel(const Fr* __restrict__ part, size_t total, unsigned S, Fr* __restrict__ out) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < total; g += (size_t)gridDim.x * blockDim.x) {
        Fr acc = fr_load(part + g);
        for (unsigned s = 1; s < S; ++s) acc = fr_add(acc, fr_load(part + s * total + g));
        fr_store(out + g, acc);
    }
}

// Full MLE evaluation: sum_i a[i] * Elo[i & (L-1)] * Ehi[i >> kl].  Each block
// takes whole chunks of L elements so that the Ehi factor is applied once per
// chunk and thread; block partials go to `partial`.
__global__ void __launch_bounds__(kThreads) fr_mle_kernel(const Fr* __restrict__ a, size_t n,
                                                           const Fr* __restrict__ Elo, unsigned kl,
                                                           const Fr* __restrict__ Ehi, Fr* __restrict__ partial) {
    __shared__ Fr red[32];
    const size_t L = (size_t)1 << kl;
    const size_t nchunks = (n + L - 1) >> kl;
    Fr acc = fr_zero();
    for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const size_t base = c << kl;
        LazyDot dot;
        dot.init();
        for (size_t j = threadIdx.x; j < L && base + j < n; j += blockDim.x) dot.add(fr_load(a + base + j), fr_load(Elo + j));
        Fr part = dot.finish();
        if (Ehi) part = fr_mmul(part, fr_load(Ehi + c));
        acc = fr_add(acc, part);
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) fr_store(partial + blockIdx.x, acc);
}

static constexpr unsigned kEqLoBits = 12;   // low table: at most 4096 entries (128 KiB, L1/L2 resident)

// d_out[0] = MLE of (d_a, n) at u; all device work on `stream`, no sync.
static int mle_eval_device(const Fr* d_a, size_t n, const zkb_fr_t* h_u, unsigned k, Fr* d_out,
                           Scratch& scratch, cudaStream_t stream) {
    if (k > 32) return fail(ZKB_ERR_LIMIT, "mle_eval: more than 32 variables");
    const unsigned kl = k < kEqLoBits ? k : kEqLoBits;
    const unsigned kh = k - kl;
    Fr* Elo = scratch.get_n<Fr>((size_t)1 << kl);
    Fr* Ehi = kh ? scratch.get_n<Fr>((size_t)1 << kh) : nullptr;
    if (!Elo || (kh && !Ehi)) return ZKB_ERR_CUDA;
    ZKB_TRY(build_eq_table(h_u, kl, Elo, stream));
    if (kh) ZKB_TRY(build_eq_table(h_u + kl, kh, Ehi, stream));
    const size_t nchunks = (n + ((size_t)1 << kl) - 1) >> kl;
    const unsigned grid = grid_for(nchunks, 1, 4);
    Fr* partial = scratch.get_n<Fr>(grid);
    if (!partial) return ZKB_ERR_CUDA;
    ZKB_LAUNCH(fr_mle_kernel, grid, kThreads, 0, stream, d_a, n, Elo, kl, Ehi, partial);
    return launch_final_sum(partial, grid, d_out, stream);
}

// d_out[other*window] = fold of the middle axis; see zkb_fr_partial_me.
int partial_me_device(const Fr* d_a, size_t a_len, size_t other, size_t J, size_t window,
                      const zkb_fr_t* h_u, unsigned k, Fr* d_out, Scratch& scratch, cudaStream_t stream) {
    if (k > 24) return fail(ZKB_ERR_LIMIT, "partial_me: folded axis longer than 2^24");
    Fr* E = scratch.get_n<Fr>((size_t)1 << k);
    if (!E) return ZKB_ERR_CUDA;
    ZKB_TRY(build_eq_table(h_u, k, E, stream));
    if (window == 1 && (other * J) <= a_len) {
        if (other >= (size_t)sm_count() * 16) {
            // enough (row, part) units for several waves of warps, parts of at least 512 entries
            unsigned parts = 1;
            while (parts < 8 && other * parts < (size_t)sm_count() * 128 && J / (parts * 2) >= 512) parts *= 2;
            if (parts == 1) {
                ZKB_LAUNCH(fr_rowdot_warp_kernel, grid_for(other, kThreads / 32, 8), kThreads, 0, stream, d_a, E, other, J, 1u, d_out);
                return ZKB_OK;
            }
            Fr* part = scratch.get_n<Fr>(other * parts);
            if (!part) return ZKB_ERR_CUDA;
            ZKB_LAUNCH(fr_rowdot_warp_kernel, grid_for(other * parts, kThreads / 32, 8), kThreads, 0, stream, d_a, E, other, J, parts, part);
            ZKB_LAUNCH(fr_sum_slices_kernel, grid_for(other, kThreads), kThreads, 0, stream, part, other, parts, d_out);
            return ZKB_OK;
        }
        ZKB_LAUNCH(fr_rowdot_kernel, grid_for(other, 1, 8), kThreads, 0, stream, d_a, E, other, J, d_out);
        return ZKB_OK;
    }
    const size_t total = other * window;
    unsigned gx = grid_for(total, kThreads, 4);
    // split the folded axis when there are too few outputs to fill the GPU
    unsigned split = 1;
    const size_t want = (size_t)sm_count() * 4;
    if (gx < want && J >= 64) {
        split = (unsigned)((want + gx - 1) / gx);
        if (split > J / 4) split = (unsigned)(J / 4);        // slices of at least four terms
        if (split < 1) split = 1;
        if (split > 64) split = 64;
    }
    if (split == 1) {
        ZKB_LAUNCH(fr_coldot_kernel, dim3(gx, 1), kThreads, 0, stream, d_a, E, other, J, window, a_len, d_out);
        return ZKB_OK;
    }
    Fr* part = scratch.get_n<Fr>(total * split);
    if (!part) return ZKB_ERR_CUDA;
    ZKB_LAUNCH(fr_coldot_kernel, dim3(gx, split), kThreads, 0, stream, d_a, E, other, J, window, a_len, part);
    ZKB_LAUNCH(fr_sum_slices_kernel, grid_for(total, kThreads), kThreads, 0, stream, part, total, split, d_out);
    return ZKB_OK;
}

// ---------------------------------------------------------------------------
// layout
// ---------------------------------------------------------------------------
__global__ void fr_pad_kernel(const Fr* __restrict__ a, size_t rows, size_t last, size_t last_p, Fr pad,
                              Fr* __restrict__ out) {
    const size_t n = rows * last_p;
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < n; g += (size_t)gridDim.x * blockDim.x) {
        const size_t r = g / last_p, c = g % last_p;
        fr_store(out + g, c < last ? fr_load(a + r * last + c) : pad);
    }
}
// 32x32 tile transpose through shared memory (coalesced both ways)
__global__ void fr_transpose_kernel(const Fr* __restrict__ a, size_t M, size_t N, Fr* __restrict__ out) {
    __shared__ Fr tile[32][33];
    const size_t bx = blockIdx.x * 32, by = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const size_t row = by + r, col = bx + threadIdx.x;
        if (row < M && col < N) tile[r][threadIdx.x] = fr_load(a + row * N + col);
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const size_t row = bx + r, col = by + threadIdx.x;   // in the transposed matrix [N, M]
        if (row < N && col < M) fr_store(out + row * M + col, tile[threadIdx.x][r]);
    }
}
// Fr_split_by_window (fr-tensor.cu:562-573): even and odd windows to two arrays
__global__ void fr_split_window_kernel(const Fr* __restrict__ a, size_t n, size_t window, Fr* __restrict__ o0, Fr* __restrict__ o1,
                                       size_t out_n) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < out_n; g += (size_t)gridDim.x * blockDim.x) {
        const size_t w = g / window, k = g % window;
        const size_t i0 = 2 * w * window + k, i1 = (2 * w + 1) * window + k;
        fr_store(o0 + g, i0 < n ? fr_load(a + i0) : fr_zero());
        fr_store(o1 + g, i1 < n ? fr_load(a + i1) : fr_zero());
    }
}
__global__ void fr_add_bias_kernel(Fr* __restrict__ z, const Fr* __restrict__ bias, size_t rows, size_t cols) {
    const size_t n = rows * cols;
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < n; g += (size_t)gridDim.x * blockDim.x)
        fr_store(z + g, fr_add(fr_load(z + g), fr_load(bias + g % cols)));
}
__global__ void fr_gather_kernel(const uint32_t* __restrict__ idx, const Fr* __restrict__ vals, Fr* __restrict__ out, size_t n) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < n; g += (size_t)gridDim.x * blockDim.x)
        fr_store(out + g, fr_load(vals + idx[g]));
}

// ---------------------------------------------------------------------------
// matmul: C[M,P] = A[M,N] * B[N,P].  32x32 output tile per block of 16x16
// threads, each thread owning a 2x2 micro-tile; the inner products are summed as
// Montgomery products (each a*b/R) and multiplied by R^2 once per output.
// ---------------------------------------------------------------------------
static constexpr int kMmTile = 32, kMmK = 16;
__global__ void __launch_bounds__(256) fr_matmul_kernel(const Fr* __restrict__ A, const Fr* __restrict__ B,
                                                         Fr* __restrict__ C, size_t M, size_t N, size_t P) {
    __shared__ Fr As[kMmTile][kMmK];
    __shared__ Fr Bs[kMmK][kMmTile];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t row0 = (size_t)blockIdx.y * kMmTile, col0 = (size_t)blockIdx.x * kMmTile;
    Fr acc[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j] = fr_zero();
    for (size_t k0 = 0; k0 < N; k0 += kMmK) {
        // A tile: 32 rows x 16 k  (512 elements, 2 per thread); B tile: 16 k x 32 cols
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int la = threadIdx.x + e * 256;
            const int ar = la >> 4, ak = la & 15;
            const size_t gr = row0 + ar, gk = k0 + ak;
            As[ar][ak] = (gr < M && gk < N) ? fr_load(A + gr * N + gk) : fr_zero();
            const int bk = la >> 5, bc = la & 31;
            const size_t gk2 = k0 + bk, gc = col0 + bc;
            Bs[bk][bc] = (gk2 < N && gc < P) ? fr_load(B + gk2 * P + gc) : fr_zero();
        }
        __syncthreads();
#pragma unroll 1
        for (int kk = 0; kk < kMmK; ++kk) {
            const Fr a0 = As[ty][kk], a1 = As[ty + 16][kk];
            const Fr b0 = Bs[kk][tx], b1 = Bs[kk][tx + 16];
            acc[0][0] = fr_add(acc[0][0], fr_mmul(a0, b0));
            acc[0][1] = fr_add(acc[0][1], fr_mmul(a0, b1));
            acc[1][0] = fr_add(acc[1][0], fr_mmul(a1, b0));
            acc[1][1] = fr_add(acc[1][1], fr_mmul(a1, b1));
        }
        __syncthreads();
    }
    const Fr r2 = fe_r2<FrP>();
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const size_t r = row0 + ty + 16 * i, c = col0 + tx + 16 * j;
            if (r < M && c < P) fr_store(C + r * P + c, fr_mmul(acc[i][j], r2));
        }
}

// ---------------------------------------------------------------------------
// 1/(a + beta) with one inversion per block (Montgomery's trick).
// Values are treated as Montgomery forms of v/R, so no conversion is needed on
// the way in; the block inverse is scaled by R^-2 once, which lands every
// output in standard form.  A zero maps to zero, as with the reference's
// exponentiation-based inverse.
// ---------------------------------------------------------------------------
static constexpr int kInvPerThread = 8;
__global__ void __launch_bounds__(kThreads) fr_inv_shifted_kernel(const Fr* __restrict__ a, Fr beta, Fr* __restrict__ out, size_t n) {
    __shared__ Fr pre[kThreads];    // inclusive prefix products over threads
    __shared__ Fr suf[kThreads];    // inclusive suffix products over threads
    __shared__ Fr inv_total;
    const size_t tile = (size_t)kThreads * kInvPerThread;
    Fr one = fr_zero();
    one.v[0] = 1;
    for (size_t base = blockIdx.x * tile; base < n; base += (size_t)gridDim.x * tile) {
        Fr x[kInvPerThread], p[kInvPerThread];
        unsigned zero_mask = 0;
#pragma unroll
        for (int e = 0; e < kInvPerThread; ++e) {
            const size_t i = base + (size_t)e * kThreads + threadIdx.x;
            Fr v = one;
            if (i < n) {
                v = fr_add(fr_load(a + i), beta);
                if (fe_is_zero(v)) { zero_mask |= 1u << e; v = one; }
            }
            x[e] = v;
            p[e] = e ? fr_mmul(p[e - 1], v) : v;
        }
        pre[threadIdx.x] = p[kInvPerThread - 1];
        suf[threadIdx.x] = p[kInvPerThread - 1];
        __syncthreads();
        // Hillis-Steele scans in both directions
        for (int off = 1; off < (int)kThreads; off <<= 1) {
            Fr np = pre[threadIdx.x], ns = suf[threadIdx.x];
            const bool hp = (int)threadIdx.x >= off, hs = threadIdx.x + off < kThreads;
            if (hp) np = fr_mmul(np, pre[threadIdx.x - off]);
            if (hs) ns = fr_mmul(ns, suf[threadIdx.x + off]);
            __syncthreads();
            pre[threadIdx.x] = np;
            suf[threadIdx.x] = ns;
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            Fr t = mont_inv<FrP>(pre[kThreads - 1]);
            t = fr_mmul(fr_mmul(t, one), one);     // * R^-2
            inv_total = t;
        }
        __syncthreads();
        // inverse of this thread's own product: inv_total * prod(other threads)
        Fr r = inv_total;
        if (threadIdx.x > 0) r = fr_mmul(r, pre[threadIdx.x - 1]);
        if (threadIdx.x + 1 < kThreads) r = fr_mmul(r, suf[threadIdx.x + 1]);
#pragma unroll
        for (int e = kInvPerThread - 1; e >= 0; --e) {
            const size_t i = base + (size_t)e * kThreads + threadIdx.x;
            Fr inv_e = e ? fr_mmul(r, p[e - 1]) : r;
            if (e) r = fr_mmul(r, x[e]);
            if (i < n) fr_store(out + i, ((zero_mask >> e) & 1u) ? fr_zero() : inv_e);
        }
        __syncthreads();
    }
}


// Same result with a long run per thread: prefix products are parked in `out`
// (which therefore must not alias `a`) instead of registers, so one inversion
// serves kInvLong * 256 elements and the kernel needs few registers, which lets
// several CTAs share an SM and hide the single-thread inversion of each other.
static constexpr int kInvLong = 32;
__global__ void __launch_bounds__(kThreads) fr_inv_shifted_long_kernel(const Fr* __restrict__ a, Fr beta, Fr* __restrict__ out, size_t n) {
    __shared__ Fr pre[kThreads];
    __shared__ Fr suf[kThreads];
    __shared__ Fr inv_total;
    const size_t tile = (size_t)kThreads * kInvLong;
    Fr one = fr_zero();
    one.v[0] = 1;
    for (size_t base = blockIdx.x * tile; base < n; base += (size_t)gridDim.x * tile) {
        Fr run = one;
#pragma unroll 1
        for (int e = 0; e < kInvLong; ++e) {
            const size_t i = base + (size_t)e * kThreads + threadIdx.x;
            if (i < n) {
                Fr v = fr_add(fr_load(a + i), beta);
                if (fe_is_zero(v)) v = one;
                run = fr_mmul(run, v);          // the run starts from the integer 1, i.e. the Montgomery form of 1/R
                fr_store(out + i, run);
            }
        }
        pre[threadIdx.x] = run;
        suf[threadIdx.x] = run;
        __syncthreads();
        for (int off = 1; off < (int)kThreads; off <<= 1) {
            Fr np = pre[threadIdx.x], ns = suf[threadIdx.x];
            if ((int)threadIdx.x >= off) np = fr_mmul(np, pre[threadIdx.x - off]);
            if (threadIdx.x + off < kThreads) ns = fr_mmul(ns, suf[threadIdx.x + off]);
            __syncthreads();
            pre[threadIdx.x] = np;
            suf[threadIdx.x] = ns;
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            Fr t = mont_inv<FrP>(pre[kThreads - 1]);
            inv_total = fr_mmul(fr_mmul(t, one), one);   // * R^-2: every inverse below comes out in standard form
        }
        __syncthreads();
        // Montgomery-domain inverse of this thread's run product
        Fr r = inv_total;
        if (threadIdx.x > 0) r = fr_mmul(r, pre[threadIdx.x - 1]);
        if (threadIdx.x + 1 < kThreads) r = fr_mmul(r, suf[threadIdx.x + 1]);
#pragma unroll 1
        for (int e = kInvLong - 1; e >= 0; --e) {
            const size_t i = base + (size_t)e * kThreads + threadIdx.x;
            if (i >= n) continue;
            Fr v = fr_add(fr_load(a + i), beta);
            const bool was_zero = fe_is_zero(v);
            if (was_zero) v = one;
            // r = 1/(run_e) in the Montgomery domain; run_(e-1) is parked one stride back
            Fr prev = e ? fr_load(out + i - kThreads) : one;
            Fr inv_e = fr_mmul(r, prev);
            r = fr_mmul(r, v);
            fr_store(out + i, was_zero ? fr_zero() : inv_e);
        }
        __syncthreads();
    }
}


// ---------------------------------------------------------------------------
// Exact integer fast path of the matmul.  Fixed-point activations and weights
// are field encodings of small signed integers; when every entry of both
// operands is such an encoding of an int32 and |a|max * |b|max * N < 2^62, the
// product is computed in int64 (32x32->64 multiply-adds) and encoded back,
// which gives the same field elements as the Montgomery path at a fraction of
// the multiply-adds.
// ---------------------------------------------------------------------------
// flags[0] = 1 if some entry is not an int32 encoding, flags[1] = max |value|
__global__ void fr_to_small_kernel(const Fr* __restrict__ a, size_t n, int32_t* __restrict__ out, unsigned* __restrict__ flags) {
    unsigned mx = 0, bad = 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const Fr x = fr_load(a + i);
        const uint32_t hi = x.v[1] | x.v[2] | x.v[3] | x.v[4] | x.v[5] | x.v[6] | x.v[7];
        int32_t v = 0;
        if (!hi && !(x.v[0] >> 31)) {
            v = (int32_t)x.v[0];
            mx = max(mx, x.v[0]);
        } else {
            const Fr m = fr_neg(x);
            const uint32_t mhi = m.v[1] | m.v[2] | m.v[3] | m.v[4] | m.v[5] | m.v[6] | m.v[7];
            if (!mhi && m.v[0] <= 0x80000000u && m.v[0] != 0) {
                v = (int32_t)(0u - m.v[0]);
                mx = max(mx, m.v[0]);
            } else {
                bad = 1;
            }
        }
        out[i] = v;
    }
    if (bad) atomicOr(flags, 1u);
    if (mx) atomicMax(flags + 1, mx);
}

// Wider left operand (softmax output times V: entries beyond int32, rows that
// sum to about the output scale).  One CTA per row: every entry with |v| < 2^61
// is split as v = hi * 2^31 + lo with lo in [-2^30, 2^30); wflags[0] = 1 if some
// entry is out of range, wl1 = the largest row sum of |hi|.
__global__ void __launch_bounds__(256) fr_to_wide_kernel(const Fr* __restrict__ a, size_t cols, int32_t* __restrict__ lo,
                                                          int32_t* __restrict__ hi, unsigned* __restrict__ wflags,
                                                          unsigned long long* __restrict__ wl1) {
    __shared__ unsigned long long red[256];
    const size_t row = blockIdx.x;
    unsigned long long l1 = 0;
    unsigned bad = 0;
    for (size_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const Fr x = fr_load(a + row * cols + c);
        long long v = 0;
        const Fr m = fr_neg(x);
        if (fr_fits_u64(x) && !(x.v[1] >> 29)) v = (long long)(((unsigned long long)x.v[1] << 32) | x.v[0]);
        else if (fr_fits_u64(m) && !(m.v[1] >> 29)) v = -(long long)(((unsigned long long)m.v[1] << 32) | m.v[0]);
        else bad = 1;
        const long long l = ((v + (1ll << 30)) & ((1ll << 31) - 1)) - (1ll << 30);
        const long long h = (v - l) >> 31;   // exact: v - l is a multiple of 2^31
        lo[row * cols + c] = (int32_t)l;
        hi[row * cols + c] = (int32_t)h;
        l1 += (unsigned long long)(h < 0 ? -h : h);
    }
    red[threadIdx.x] = l1;
    __syncthreads();
    for (unsigned st = 128; st > 0; st >>= 1) {
        if (threadIdx.x < st) red[threadIdx.x] += red[threadIdx.x + st];
        __syncthreads();
    }
    if (threadIdx.x == 0) atomicMax(wl1, red[0]);
    if (bad) atomicOr(wflags, 1u);
}

// acc_hi * 2^31 + acc_lo as a field element (|acc_hi|, |acc_lo| < 2^62)
ZKB_DEV Fr fr_from_split(long long acc_lo, long long acc_hi) {
    const unsigned long long mag = acc_hi < 0 ? 0ull - (unsigned long long)acc_hi : (unsigned long long)acc_hi;
    Fr r = fr_zero();
    // mag << 31 over three limbs
    r.v[0] = (uint32_t)(mag << 31);
    r.v[1] = (uint32_t)(mag >> 1);
    r.v[2] = (uint32_t)(mag >> 33);
    if (acc_hi < 0) r = fr_neg(r);
    return fr_add(r, fr_from_i64(acc_lo));
}

// ---- exact integer matmul on the tensor cores, through 8-bit limbs -------------------------
// For a left operand below 2^23 and a right operand below 2^15 in magnitude (activations times weights: the six
// linear layers of a decoder layer), A = a2 2^16 + a1 2^8 + a0 and B = b1 2^8 + b0 with a0, a1, b0 in [0, 255] and
// a2, b1 signed bytes, and A B = sum_{i,j} 2^(8(i+j)) a_i b_j: six 8-bit products with 32-bit accumulators
// (mma.sync m16n8k32, the integer tensor-core instruction; |a_i b_j| <= 255^2 per term, so two products of one weight
// 2^(8c) share an accumulator for up to 16384 terms).  Exact: the epilogue recombines the four accumulators in 64 bits.
static constexpr int kI8TileM = 128, kI8TileP = 64, kI8TileK = 64, kI8Pitch = 80;   // pitch: 64 bytes + 16, conflict-free
static constexpr size_t kI8MaxK = 16384;

// A [M][K] int32 -> three byte planes [M][Kp], zero padded to Kp (a multiple of 64)
__global__ void i8_split_rows_kernel(const int32_t* __restrict__ a, size_t M, size_t K, size_t Kp, uint8_t* __restrict__ p0,
                                     uint8_t* __restrict__ p1, int8_t* __restrict__ p2) {
    const size_t total = M * Kp;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const size_t r = t / Kp, k = t % Kp;
        const int v = k < K ? a[r * K + k] : 0;
        p0[t] = (uint8_t)(v & 255);
        p1[t] = (uint8_t)((v >> 8) & 255);
        p2[t] = (int8_t)(v >> 16);             // arithmetic shift: the signed top limb
    }
}
// B [K][P] int32 -> two byte planes of the transpose [P][Kp]
__global__ void i8_split_cols_kernel(const int32_t* __restrict__ b, size_t K, size_t P, size_t Kp, uint8_t* __restrict__ p0,
                                     int8_t* __restrict__ p1) {
    __shared__ int32_t tile[32][33];
    const size_t k0 = (size_t)blockIdx.y * 32, c0 = (size_t)blockIdx.x * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const size_t k = k0 + j, c = c0 + threadIdx.x;
        tile[j][threadIdx.x] = (k < K && c < P) ? b[k * P + c] : 0;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const size_t c = c0 + j, k = k0 + threadIdx.x;
        if (c < P && k < Kp) {
            const int v = tile[threadIdx.x][j];
            p0[c * Kp + k] = (uint8_t)(v & 255);
            p1[c * Kp + k] = (int8_t)(v >> 8);
        }
    }
}

#define ZKB_IMMA(TA, TB, acc, a, b)                                                                              \
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32." TA "." TB ".s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, " \
                 "{%0,%1,%2,%3};"                                                                                \
                 : "+r"(acc[0]), "+r"(acc[1]), "+r"(acc[2]), "+r"(acc[3])                                        \
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]))

// One CTA: a 128 x 64 tile of C; eight warps as 4 x 2, each 32 x 32 = 2 x 4 instruction tiles, four accumulator sets.
__global__ void __launch_bounds__(256) i8_limb_matmul_kernel(const uint8_t* __restrict__ A0, const uint8_t* __restrict__ A1,
                                                              const int8_t* __restrict__ A2, const uint8_t* __restrict__ B0,
                                                              const int8_t* __restrict__ B1, Fr* __restrict__ C, size_t M,
                                                              size_t Kp, size_t P) {
    __shared__ __align__(16) uint8_t As[3][kI8TileM][kI8Pitch];
    __shared__ __align__(16) uint8_t Bs[2][kI8TileP][kI8Pitch];
    const size_t row0 = (size_t)blockIdx.y * kI8TileM, col0 = (size_t)blockIdx.x * kI8TileP;
    const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, g = lane >> 2, tig = lane & 3u;
    const unsigned wm = (warp >> 1) * 32, wp = (warp & 1u) * 32;
    int acc[4][2][4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[c][i][j][e] = 0;
    const uint8_t* Ap[3] = {A0, A1, reinterpret_cast<const uint8_t*>(A2)};
    const uint8_t* Bp[2] = {B0, reinterpret_cast<const uint8_t*>(B1)};
    for (size_t k0 = 0; k0 < Kp; k0 += kI8TileK) {
        // global -> shared, 16 bytes per access: 128 rows x 4 vectors per A plane, 64 x 4 per B plane
        for (unsigned v = threadIdx.x; v < 3 * kI8TileM * 4; v += 256) {
            const unsigned pl = v / (kI8TileM * 4), r = (v / 4) % kI8TileM, q = v & 3u;
            uint4 x = make_uint4(0, 0, 0, 0);
            if (row0 + r < M) x = *reinterpret_cast<const uint4*>(Ap[pl] + (row0 + r) * Kp + k0 + 16 * q);
            *reinterpret_cast<uint4*>(&As[pl][r][16 * q]) = x;
        }
        for (unsigned v = threadIdx.x; v < 2 * kI8TileP * 4; v += 256) {
            const unsigned pl = v / (kI8TileP * 4), r = (v / 4) % kI8TileP, q = v & 3u;
            uint4 x = make_uint4(0, 0, 0, 0);
            if (col0 + r < P) x = *reinterpret_cast<const uint4*>(Bp[pl] + (col0 + r) * Kp + k0 + 16 * q);
            *reinterpret_cast<uint4*>(&Bs[pl][r][16 * q]) = x;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kI8TileK; kk += 32) {
            unsigned a[3][2][4], b[2][4][2];
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const unsigned r = wm + 16 * i + g;
                    a[pl][i][0] = *reinterpret_cast<const unsigned*>(&As[pl][r][kk + 4 * tig]);
                    a[pl][i][1] = *reinterpret_cast<const unsigned*>(&As[pl][r + 8][kk + 4 * tig]);
                    a[pl][i][2] = *reinterpret_cast<const unsigned*>(&As[pl][r][kk + 16 + 4 * tig]);
                    a[pl][i][3] = *reinterpret_cast<const unsigned*>(&As[pl][r + 8][kk + 16 + 4 * tig]);
                }
#pragma unroll
            for (int pl = 0; pl < 2; ++pl)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned c = wp + 8 * j + g;
                    b[pl][j][0] = *reinterpret_cast<const unsigned*>(&Bs[pl][c][kk + 4 * tig]);
                    b[pl][j][1] = *reinterpret_cast<const unsigned*>(&Bs[pl][c][kk + 16 + 4 * tig]);
                }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ZKB_IMMA("u8", "u8", acc[0][i][j], a[0][i], b[0][j]);   // a0 b0
                    ZKB_IMMA("u8", "u8", acc[1][i][j], a[1][i], b[0][j]);   // a1 b0
                    ZKB_IMMA("u8", "s8", acc[1][i][j], a[0][i], b[1][j]);   // a0 b1
                    ZKB_IMMA("s8", "u8", acc[2][i][j], a[2][i], b[0][j]);   // a2 b0
                    ZKB_IMMA("u8", "s8", acc[2][i][j], a[1][i], b[1][j]);   // a1 b1
                    ZKB_IMMA("s8", "s8", acc[3][i][j], a[2][i], b[1][j]);   // a2 b1
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const size_t r = row0 + wm + 16 * i + g + ((e & 2) ? 8 : 0);
                const size_t c = col0 + wp + 8 * j + 2 * tig + (e & 1);
                if (r < M && c < P) {
                    const long long v = (long long)acc[0][i][j][e] + ((long long)acc[1][i][j][e] << 8) +
                                        ((long long)acc[2][i][j][e] << 16) + ((long long)acc[3][i][j][e] << 24);
                    fr_store(C + r * P + c, fr_from_i64(v));
                }
            }
}
#undef ZKB_IMMA

static constexpr int kImTile = 64, kImK = 16;
template <bool WIDE>
__global__ void __launch_bounds__(256) i32_matmul_kernel(const int32_t* __restrict__ A, const int32_t* __restrict__ Ahi,
                                                          const int32_t* __restrict__ B, Fr* __restrict__ C, size_t M, size_t N,
                                                          size_t P) {
    __shared__ int32_t As[kImK][kImTile + 1];   // [k][row]
    __shared__ int32_t Ah[WIDE ? kImK : 1][kImTile + 1];
    __shared__ int32_t Bs[kImK][kImTile];       // [k][col]
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t row0 = (size_t)blockIdx.y * kImTile, col0 = (size_t)blockIdx.x * kImTile;
    long long acc[4][4], acch[WIDE ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0;
            if constexpr (WIDE) acch[i][j] = 0;
        }
    for (size_t k0 = 0; k0 < N; k0 += kImK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int l = threadIdx.x + e * 256;          // 1024 elements per tile
            const int ar = l >> 4, ak = l & 15;           // A tile: 64 rows x 16 k, k fastest (coalesced along k)
            const size_t gr = row0 + ar, gk = k0 + ak;
            As[ak][ar] = (gr < M && gk < N) ? A[gr * N + gk] : 0;
            if constexpr (WIDE) Ah[ak][ar] = (gr < M && gk < N) ? Ahi[gr * N + gk] : 0;
            const int bk = l >> 6, bc = l & 63;           // B tile: 16 k x 64 cols
            const size_t gk2 = k0 + bk, gc = col0 + bc;
            Bs[bk][bc] = (gk2 < N && gc < P) ? B[gk2 * P + gc] : 0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kImK; ++kk) {
            int a[4], ah[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = As[kk][ty + 16 * i];
                if constexpr (WIDE) ah[i] = Ah[kk][ty + 16 * i]; else ah[i] = 0;
                b[i] = Bs[kk][tx + 16 * i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] += (long long)a[i] * (long long)b[j];
                    if constexpr (WIDE) acch[i][j] += (long long)ah[i] * (long long)b[j];
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t r = row0 + ty + 16 * i, c = col0 + tx + 16 * j;
            if (r < M && c < P) {
                if constexpr (WIDE) fr_store(C + r * P + c, fr_from_split(acc[i][j], acch[i][j]));
                else fr_store(C + r * P + c, fr_from_i64(acc[i][j]));
            }
        }
}

}  // namespace zkb

using namespace zkb;

#define FR(p) reinterpret_cast<Fr*>(p)
#define CFR(p) reinterpret_cast<const Fr*>(p)

static inline Fr host_to_dev(const zkb_fr_t& x) {
    Fr r;
    memcpy(r.v, x.val, 32);
    return r;
}
static inline Fr host_to_dev_mont(const zkb_fr_t& x) {
    zkb_fr_t m = hfr::store(hfr::to_mont(hfr::load(x)));
    return host_to_dev(m);
}

extern "C" {

int zkb_fr_from_i32(const int32_t* d_in, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_from_i32_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream), d_in, FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_from_i64(const int64_t* d_in, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_from_i64_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream), d_in, FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_to_i32(const zkb_fr_t* d_in, int32_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_to_i32_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream), CFR(d_in), d_out, n);
    return ZKB_OK;
}
int zkb_fr_to_i64(const zkb_fr_t* d_in, int64_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_to_i64_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream), CFR(d_in), d_out, n);
    return ZKB_OK;
}
int zkb_fr_from_f32(const float* d_in, uint64_t scale, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_from_f32_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream), d_in, (unsigned long)scale, FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_from_f64(const double* d_in, uint64_t scale, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_from_f64_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream), d_in, (unsigned long)scale, FR(d_out), n);
    return ZKB_OK;
}

#define ZKB_BINARY(name, OP)                                                                         \
    int name(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_out, size_t n, void* stream) {   \
        if (!n) return ZKB_OK;                                                                       \
        ZKB_LAUNCH(fr_binary_kernel<OP>, grid_for(n, kThreads), kThreads, 0, as_stream(stream),      \
                   CFR(d_a), CFR(d_b), FR(d_out), n);                                                \
        return ZKB_OK;                                                                               \
    }
ZKB_BINARY(zkb_fr_add, BinOp::Add)
ZKB_BINARY(zkb_fr_sub, BinOp::Sub)
ZKB_BINARY(zkb_fr_mul, BinOp::Mul)
ZKB_BINARY(zkb_fr_mont_mul, BinOp::MontMul)

int zkb_fr_add_scalar(const zkb_fr_t* d_a, const zkb_fr_t* h_x, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_scalar_kernel<BinOp::Add>, grid_for(n, kThreads), kThreads, 0, as_stream(stream),
               CFR(d_a), host_to_dev(*h_x), FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_sub_scalar(const zkb_fr_t* d_a, const zkb_fr_t* h_x, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_scalar_kernel<BinOp::Sub>, grid_for(n, kThreads), kThreads, 0, as_stream(stream),
               CFR(d_a), host_to_dev(*h_x), FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_mul_scalar(const zkb_fr_t* d_a, const zkb_fr_t* h_x, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_scalar_kernel<BinOp::Mul>, grid_for(n, kThreads), kThreads, 0, as_stream(stream),
               CFR(d_a), host_to_dev_mont(*h_x), FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_neg(const zkb_fr_t* d_a, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_unary_kernel<UnOp::Neg>, grid_for(n, kThreads), kThreads, 0, as_stream(stream), CFR(d_a), FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_mont(const zkb_fr_t* d_a, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_unary_kernel<UnOp::Mont>, grid_for(n, kThreads), kThreads, 0, as_stream(stream), CFR(d_a), FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_unmont(const zkb_fr_t* d_a, zkb_fr_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_unary_kernel<UnOp::Unmont>, grid_for(n, kThreads), kThreads, 0, as_stream(stream), CFR(d_a), FR(d_out), n);
    return ZKB_OK;
}
int zkb_fr_inv_shifted(const zkb_fr_t* d_a, const zkb_fr_t* h_beta, zkb_fr_t* d_out, size_t n, void* stream) {
    ZKB_API_RANGE();
    if (!n) return ZKB_OK;
    if (static_cast<const void*>(d_a) != static_cast<const void*>(d_out) && n >= (size_t)kThreads * kInvLong) {
        ZKB_LAUNCH(fr_inv_shifted_long_kernel, grid_for(n, kThreads * kInvLong, 8), kThreads, 0, as_stream(stream),
                   CFR(d_a), host_to_dev(*h_beta), FR(d_out), n);
        return ZKB_OK;
    }
    ZKB_LAUNCH(fr_inv_shifted_kernel, grid_for(n, kThreads * kInvPerThread, 4), kThreads, 0, as_stream(stream),
               CFR(d_a), host_to_dev(*h_beta), FR(d_out), n);
    return ZKB_OK;
}

int zkb_fr_sum(const zkb_fr_t* d_a, size_t n, zkb_fr_t* h_out, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (n == 0) { memset(h_out, 0, sizeof(*h_out)); return ZKB_OK; }
    Scratch scratch(s);
    const unsigned grid = grid_for(n, kThreads * 8, 4);
    Fr* partial = scratch.get_n<Fr>(grid + 1);
    if (!partial) return ZKB_ERR_CUDA;
    ZKB_LAUNCH(fr_partial_sum_kernel, grid, kThreads, 0, s, CFR(d_a), n, partial);
    ZKB_TRY(launch_final_sum(partial, grid, partial + grid, s));
    ZKB_CUDA(cudaMemcpyAsync(h_out, partial + grid, 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_fr_mle_eval(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k, zkb_fr_t* h_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (k > 32 || n == 0) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    const size_t full = (size_t)1 << k;
    if (n <= full / 2 || n > full) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    Scratch scratch(s);
    Fr* d_out = scratch.get_n<Fr>(1);
    if (!d_out) return ZKB_ERR_CUDA;
    ZKB_TRY(mle_eval_device(CFR(d_a), n, h_u, k, d_out, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_out, d_out, 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_fr_partial_me(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k,
                      size_t cur_dim, size_t window, zkb_fr_t* d_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (k > 31) return fail(ZKB_ERR_LIMIT, "partial_me: too many variables");
    if (cur_dim <= (((size_t)1 << k) >> 1)) return fail(ZKB_ERR_DIM, "cur_dim <= ((1<<u.size()) >> 1)");
    if (cur_dim > ((size_t)1 << k)) return fail(ZKB_ERR_DIM, "cur_dim > (1<<u.size())");
    if (window == 0 || n % (cur_dim * window) != 0) return fail(ZKB_ERR_DIM, "t.size % (cur_dim * window_size) != 0");
    if (k == 0) {   // cur_dim == 1: nothing to fold
        ZKB_CUDA(cudaMemcpyAsync(d_out, d_a, n * 32, cudaMemcpyDeviceToDevice, s));
        return ZKB_OK;
    }
    Scratch scratch(s);
    return partial_me_device(CFR(d_a), n, n / (cur_dim * window), cur_dim, window, h_u, k, FR(d_out), scratch, s);
}

int zkb_fr_partial_me_window(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k,
                             size_t window, zkb_fr_t* d_out, size_t* out_n, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (k > 31 || window == 0) return fail(ZKB_ERR_ARG, "partial_me: bad arguments");
    if (k >= 1 && n <= window * ((size_t)1 << (k - 1))) return fail(ZKB_ERR_DIM, "partial_me: Incompatible dimensions");
    const size_t J = (size_t)1 << k;
    const size_t nwin = (n + window - 1) / window;
    const size_t groups = (nwin + J - 1) / J;
    if (out_n) *out_n = groups * window;
    if (k == 0) {
        ZKB_CUDA(cudaMemcpyAsync(d_out, d_a, n * 32, cudaMemcpyDeviceToDevice, s));
        if (out_n) *out_n = n;
        return ZKB_OK;
    }
    Scratch scratch(s);
    // view as [groups, J, window] with everything past n reading as zero
    return partial_me_device(CFR(d_a), n, groups, J, window, h_u, k, FR(d_out), scratch, s);
}

int zkb_fr_mle_eval_2d(const zkb_fr_t* d_a, size_t d0, size_t d1,
                       const zkb_fr_t* h_u0, unsigned k0, const zkb_fr_t* h_u1, unsigned k1,
                       zkb_fr_t* h_out, void* stream) {
    ZKB_API_RANGE();
    cudaStream_t s = as_stream(stream);
    if (k0 > 31 || k1 > 31) return fail(ZKB_ERR_LIMIT, "multi_dim_me: too many variables");
    if (d1 <= (((size_t)1 << k1) >> 1)) return fail(ZKB_ERR_DIM, "cur_dim <= ((1<<u.size()) >> 1)");
    if (d1 > ((size_t)1 << k1)) return fail(ZKB_ERR_DIM, "cur_dim > (1<<u.size())");
    if (d0 <= (((size_t)1 << k0) / 2) || d0 > ((size_t)1 << k0)) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    Scratch scratch(s);
    Fr* rowred = scratch.get_n<Fr>(d0 + 1);
    if (!rowred) return ZKB_ERR_CUDA;
    if (k1 == 0) {
        ZKB_CUDA(cudaMemcpyAsync(rowred, d_a, d0 * 32, cudaMemcpyDeviceToDevice, s));
    } else {
        ZKB_TRY(partial_me_device(CFR(d_a), d0 * d1, d0, d1, 1, h_u1, k1, rowred, scratch, s));
    }
    ZKB_TRY(mle_eval_device(rowred, d0, h_u0, k0, rowred + d0, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_out, rowred + d0, 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

int zkb_fr_pad_last(const zkb_fr_t* d_a, size_t rows, size_t last, size_t last_padded,
                    const zkb_fr_t* h_pad_val, zkb_fr_t* d_out, void* stream) {
    if (last_padded < last) return fail(ZKB_ERR_DIM, "pad: padded extent smaller than extent");
    const size_t n = rows * last_padded;
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(fr_pad_kernel, grid_for(n, kThreads), kThreads, 0, as_stream(stream),
               CFR(d_a), rows, last, last_padded, host_to_dev(*h_pad_val), FR(d_out));
    return ZKB_OK;
}
int zkb_fr_transpose(const zkb_fr_t* d_a, size_t M, size_t N, zkb_fr_t* d_out, void* stream) {
    if (!M || !N) return ZKB_OK;
    dim3 grid(div_up(N, 32), div_up(M, 32)), block(32, 8);
    if (grid.y > 65535) return fail(ZKB_ERR_LIMIT, "transpose: more than 2^21 rows");
    ZKB_LAUNCH(fr_transpose_kernel, grid, block, 0, as_stream(stream), CFR(d_a), M, N, FR(d_out));
    return ZKB_OK;
}
int zkb_fr_matmul(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_c, size_t M, size_t N, size_t P, void* stream) {
    ZKB_API_RANGE();
    if (!M || !P) return ZKB_OK;
    cudaStream_t s = as_stream(stream);
    if (N && M * N * P >= ((size_t)1 << 22)) {
        // try the exact int64 path (worth a small device-to-host read only for large products)
        Scratch scratch(s);
        int32_t* ia = scratch.get_n<int32_t>(M * N);
        int32_t* ib = scratch.get_n<int32_t>(N * P);
        unsigned* flags = scratch.get_n<unsigned>(4);
        if (!ia || !ib || !flags) return ZKB_ERR_CUDA;
        ZKB_CUDA(cudaMemsetAsync(flags, 0, 16, s));
        ZKB_LAUNCH(fr_to_small_kernel, grid_for(M * N, kThreads), kThreads, 0, s, CFR(d_a), M * N, ia, flags);
        ZKB_LAUNCH(fr_to_small_kernel, grid_for(N * P, kThreads), kThreads, 0, s, CFR(d_b), N * P, ib, flags + 2);
        unsigned h[4];
        ZKB_CUDA(cudaMemcpyAsync(h, flags, 16, cudaMemcpyDeviceToHost, s));
        ZKB_CUDA(cudaStreamSynchronize(s));
        // |sum| <= N * maxA * maxB must stay below 2^62
        const unsigned __int128 bound = (unsigned __int128)h[1] * h[3] * N;
        const unsigned __int128 limit = (unsigned __int128)1 << 62;
        dim3 gi(div_up(P, kImTile), div_up(M, kImTile));
        if (gi.y > 65535) return fail(ZKB_ERR_LIMIT, "matmul: more than 2^22 rows");
        if (!h[0] && !h[2] && h[1] < (1u << 23) && h[3] < (1u << 15) && N <= kI8MaxK && M * N * P >= ((size_t)1 << 27)) {
            // both operands short enough for 8-bit limbs: the tensor-core path
            const size_t Kp = (N + kI8TileK - 1) / kI8TileK * kI8TileK;
            uint8_t* pa = scratch.get_n<uint8_t>(3 * M * Kp);
            uint8_t* pb = scratch.get_n<uint8_t>(2 * P * Kp);
            if (!pa || !pb) return ZKB_ERR_CUDA;
            dim3 gt(div_up(P, 32), div_up(Kp, 32)), g8(div_up(P, kI8TileP), div_up(M, kI8TileM));
            if (gt.y > 65535 || g8.y > 65535) return fail(ZKB_ERR_LIMIT, "matmul: more than 2^22 rows");
            ZKB_LAUNCH(i8_split_rows_kernel, grid_for(M * Kp, kThreads), kThreads, 0, s, ia, M, N, Kp, pa, pa + M * Kp,
                       reinterpret_cast<int8_t*>(pa + 2 * M * Kp));
            ZKB_LAUNCH(i8_split_cols_kernel, gt, dim3(32, 8), 0, s, ib, N, P, Kp, pb, reinterpret_cast<int8_t*>(pb + P * Kp));
            ZKB_LAUNCH(i8_limb_matmul_kernel, g8, 256, 0, s, pa, pa + M * Kp, reinterpret_cast<const int8_t*>(pa + 2 * M * Kp), pb,
                       reinterpret_cast<const int8_t*>(pb + P * Kp), FR(d_c), M, Kp, P);
            return ZKB_OK;
        }
        if (!h[0] && !h[2] && bound < limit) {
            ZKB_LAUNCH(i32_matmul_kernel<false>, gi, 256, 0, s, ia, nullptr, ib, FR(d_c), M, N, P);
            return ZKB_OK;
        }
        if (!h[2] && M <= 0x7fffffffull) {
            // left operand beyond int32: two 31-bit halves, the high half bounded by its row sums
            int32_t* ih = scratch.get_n<int32_t>(M * N);
            unsigned long long* wl1 = scratch.get_n<unsigned long long>(2);
            if (!ih || !wl1) return ZKB_ERR_CUDA;
            ZKB_CUDA(cudaMemsetAsync(wl1, 0, 16, s));
            ZKB_LAUNCH(fr_to_wide_kernel, (unsigned)M, 256, 0, s, CFR(d_a), N, ia, ih, reinterpret_cast<unsigned*>(wl1 + 1), wl1);
            unsigned long long hw[2];
            ZKB_CUDA(cudaMemcpyAsync(hw, wl1, 16, cudaMemcpyDeviceToHost, s));
            ZKB_CUDA(cudaStreamSynchronize(s));
            const unsigned __int128 lo_bound = ((unsigned __int128)N << 30) * h[3];
            const unsigned __int128 hi_bound = (unsigned __int128)hw[0] * h[3];
            if (!(hw[1] & 1u) && lo_bound < limit && hi_bound < limit) {
                ZKB_LAUNCH(i32_matmul_kernel<true>, gi, 256, 0, s, ia, ih, ib, FR(d_c), M, N, P);
                return ZKB_OK;
            }
        }
    }
    dim3 grid(div_up(P, kMmTile), div_up(M, kMmTile));
    if (grid.y > 65535) return fail(ZKB_ERR_LIMIT, "matmul: more than 2^21 rows");
    ZKB_LAUNCH(fr_matmul_kernel, grid, 256, 0, s, CFR(d_a), CFR(d_b), FR(d_c), M, N, P);
    return ZKB_OK;
}
int zkb_fr_split_window(const zkb_fr_t* d_a, size_t n, size_t window, zkb_fr_t* d_out0, zkb_fr_t* d_out1, size_t out_n, void* stream) {
    if (!out_n) return ZKB_OK;
    if (!window) return fail(ZKB_ERR_ARG, "Invalid window size.");
    ZKB_LAUNCH(fr_split_window_kernel, grid_for(out_n, kThreads), kThreads, 0, as_stream(stream),
               CFR(d_a), n, window, FR(d_out0), FR(d_out1), out_n);
    return ZKB_OK;
}
int zkb_fr_add_bias(zkb_fr_t* d_z, const zkb_fr_t* d_bias, size_t rows, size_t cols, void* stream) {
    if (!rows || !cols) return ZKB_OK;
    ZKB_LAUNCH(fr_add_bias_kernel, grid_for(rows * cols, kThreads), kThreads, 0, as_stream(stream),
               FR(d_z), CFR(d_bias), rows, cols);
    return ZKB_OK;
}
int zkb_fr_gather(const uint32_t* d_indices, const zkb_fr_t* d_vals, zkb_fr_t* d_out, size_t D, void* stream) {
    if (!D) return ZKB_OK;
    ZKB_LAUNCH(fr_gather_kernel, grid_for(D, kThreads), kThreads, 0, as_stream(stream), d_indices, CFR(d_vals), FR(d_out), D);
    return ZKB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// zkb_fr_mle_eval_noalloc: the same evaluation as zkb_fr_mle_eval for callers
// that must not allocate device memory.  Examples: a host process that handed
// the whole GPU to its own memory manager at start-up and cannot let a library
// take memory behind its back, or a latency-critical loop that cannot afford the
// allocator's locks.  The eq-tables, the per-CTA partial sums and the result
// slot live in one file-scope device array of fixed size instead of pool
// blocks; nothing here calls cudaMalloc, cudaFree, the stream-ordered pool or
// any other allocating routine.
// ---------------------------------------------------------------------------
static constexpr unsigned kNoAllocMaxVars = 24;                       // n <= 2^24 elements
static constexpr unsigned kNoAllocGrid = 1024;                        // at most this many partial sums
static constexpr size_t kNoAllocLo = (size_t)1 << kEqLoBits;          // 4096-entry low table
static constexpr size_t kNoAllocHi = (size_t)1 << (kNoAllocMaxVars - kEqLoBits);
static constexpr size_t kNoAllocElems = kNoAllocLo + kNoAllocHi + kNoAllocGrid + 1;   // 9217 Fr = 288 KiB per GPU
static __device__ __align__(256) zkb::Fr g_noalloc_scratch[kNoAllocElems];

// The array's name is a host-side stand-in in host code, not a device address:
// the address the kernels need is looked up once per device and kept (atomically:
// two host threads may make their first call at the same time; both look up the
// same address).  A cudaDeviceReset in the same process invalidates the kept address.
static std::atomic<zkb::Fr*> g_noalloc_addr[64];

static int noalloc_scratch(zkb::Fr** out) {
    int dev = 0;
    ZKB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(ZKB_ERR_LIMIT, "zkb_fr_mle_eval_noalloc: device index above 63");
    zkb::Fr* addr = g_noalloc_addr[dev].load(std::memory_order_acquire);
    if (!addr) {
        void* p = nullptr;
        ZKB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        addr = static_cast<zkb::Fr*>(p);
        g_noalloc_addr[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return ZKB_OK;
}

#define ZKB_LAUNCH_NOALLOC(kernel, grid, block, stream, ...)              \
    do {                                                                  \
        kernel<<<(grid), (block), 0, (stream)>>>(__VA_ARGS__);            \
        ::zkb::g_launches.fetch_add(1, std::memory_order_relaxed);        \
        ZKB_LAUNCH_CHECK(#kernel);                                        \
    } while (0)

extern "C" int zkb_fr_mle_eval_noalloc(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k, zkb_fr_t* h_out, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (k > kNoAllocMaxVars || n > ((size_t)1 << kNoAllocMaxVars))
        return fail(ZKB_ERR_LIMIT, "zkb_fr_mle_eval_noalloc: at most 2^24 elements (24 variables); use zkb_fr_mle_eval for larger tensors");
    if (n == 0) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    const size_t full = (size_t)1 << k;
    if (n <= full / 2 || n > full) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    Fr* base = nullptr;
    ZKB_TRY(noalloc_scratch(&base));
    Fr* lo = base;
    Fr* hi = base + kNoAllocLo;
    Fr* partial = hi + kNoAllocHi;
    Fr* result = partial + kNoAllocGrid;
    const unsigned kl = k < kEqLoBits ? k : kEqLoBits, kh = k - kl;
    Challenges ch;
    memset(&ch, 0, sizeof(ch));
    for (unsigned j = 0; j < kl; ++j) memcpy(ch.u[j].v, h_u[j].val, 32);
    ZKB_LAUNCH_NOALLOC(eq_table_kernel, grid_for((size_t)1 << kl, kThreads), kThreads, s, ch, kl, lo);
    if (kh) {
        memset(&ch, 0, sizeof(ch));
        for (unsigned j = 0; j < kh; ++j) memcpy(ch.u[j].v, h_u[kl + j].val, 32);
        ZKB_LAUNCH_NOALLOC(eq_table_kernel, grid_for((size_t)1 << kh, kThreads), kThreads, s, ch, kh, hi);
    }
    const size_t nchunks = (n + ((size_t)1 << kl) - 1) >> kl;
    unsigned grid = grid_for(nchunks, 1, 4);
    if (grid > kNoAllocGrid) grid = kNoAllocGrid;
    // every slot that is read below is written first by this call: nothing has to start at zero
    ZKB_LAUNCH_NOALLOC(fr_mle_kernel, grid, kThreads, s, CFR(d_a), n, lo, kl, kh ? hi : nullptr, partial);
    ZKB_LAUNCH_NOALLOC(fr_final_sum_kernel, 1, kThreads, s, partial, (size_t)grid, result);
    ZKB_CUDA(cudaMemcpyAsync(h_out, result, 32, cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}
