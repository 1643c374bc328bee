// G1 tensor device work: elementwise group operations, affine normalisation,
// scalar multiplication, sums, the multilinear fold in the exponent and the
// (the opening rounds of the commitment, me_open, live beside the MSM).
#include "frutil.cuh"
#include "g1.cuh"
#include "hostfr.hpp"

#include <vector>

namespace zkb {

static constexpr unsigned kG1Threads = 128;

enum class G1Bin { Add, Sub };

template <G1Bin OP>
__global__ void __launch_bounds__(kG1Threads) g1_binary_kernel(const G1Jac* __restrict__ a, const G1Jac* __restrict__ b,
                                                                G1Jac* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        G1Jac x = g1_load(a + i), y = g1_load(b + i);
        if (OP == G1Bin::Sub) y = g1_neg(y);
        g1_store(out + i, g1_add(x, y));
    }
}
__global__ void __launch_bounds__(kG1Threads) g1_add_scalar_kernel(const G1Jac* __restrict__ a, G1Jac y, G1Jac* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        g1_store(out + i, g1_add(g1_load(a + i), y));
}
__global__ void g1_neg_kernel(const G1Jac* __restrict__ a, G1Jac* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        g1_store(out + i, g1_neg(g1_load(a + i)));
}
__global__ void g1_fill_kernel(G1Jac* __restrict__ out, G1Jac v, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        g1_store(out + i, v);
}
__global__ void g1_from_affine_kernel(const G1Aff* __restrict__ a, G1Jac* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const G1Aff p = g1_aff_load(a + i);
        G1Jac r;
        r.x = p.x; r.y = p.y; r.z = fe_mont_one<FqParams>();   // as the reference: Z = 1 always
        g1_store(out + i, r);
    }
}

// Jacobian -> affine with one field inversion per thread.
__global__ void __launch_bounds__(kG1Threads) g1_to_affine_kernel(const G1Jac* __restrict__ a, G1Aff* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const G1Jac p = g1_load(a + i);
        G1Aff r;
        if (g1_is_identity(p)) {
            r.x = fe_zero<FqParams>(); r.y = fe_zero<FqParams>();
        } else {
            const Fq zi = mont_inv<FqParams>(p.z);
            const Fq zi2 = fq_sqr(zi);
            r.x = fq_mul(p.x, zi2);
            r.y = fq_mul(p.y, fq_mul(zi2, zi));
        }
        g1_aff_store(out + i, r);
    }
}

__global__ void __launch_bounds__(kG1Threads) g1_mul_kernel(const G1Jac* __restrict__ g, size_t n_g, const Fr* __restrict__ k,
                                                             size_t n, G1Jac* __restrict__ out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        g1_store(out + i, g1_mul_bits(g1_load(g + i % n_g), fr_load(k + i)));
}

// Block-level tree sum in shared memory (blockDim.x Jacobian points).
ZKB_DEV G1Jac g1_block_sum(G1Jac v, G1Jac* smem) {
    smem[threadIdx.x] = v;
    __syncthreads();
    for (unsigned s = blockDim.x >> 1; s > 0; s >>= 1) {
        if (threadIdx.x < s) smem[threadIdx.x] = g1_add(smem[threadIdx.x], smem[threadIdx.x + s]);
        __syncthreads();
    }
    G1Jac r = smem[0];
    __syncthreads();
    return r;
}
static constexpr unsigned kSumThreads = 64;
// out[row * gridDim.x + blockIdx.x] = partial sum of row `row` (cols strided over the grid's x blocks)
__global__ void __launch_bounds__(kSumThreads) g1_row_partial_sum_kernel(const G1Jac* __restrict__ a, size_t cols,
                                                                          G1Jac* __restrict__ out) {
    __shared__ G1Jac sm[kSumThreads];
    const size_t row = blockIdx.y;
    G1Jac acc = g1_identity();
    for (size_t c = blockIdx.x * (size_t)blockDim.x + threadIdx.x; c < cols; c += (size_t)gridDim.x * blockDim.x)
        acc = g1_add(acc, g1_load(a + row * cols + c));
    acc = g1_block_sum(acc, sm);
    if (threadIdx.x == 0) g1_store(out + row * gridDim.x + blockIdx.x, acc);
}

// One round of the fold in the exponent (G1_me_step, g1-tensor.cu:486-497):
// out[g] = a[2g] + x*(a[2g+1] - a[2g]) with x given as raw scalar bits.
__global__ void __launch_bounds__(kG1Threads) g1_me_step_kernel(const G1Jac* __restrict__ a, size_t n_in, size_t n_out,
                                                                 Fr x_bits, G1Jac* __restrict__ out) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < n_out; g += (size_t)gridDim.x * blockDim.x) {
        const G1Jac p0 = g1_load(a + 2 * g);
        G1Jac r;
        if (2 * g + 1 < n_in) {
            const G1Jac p1 = g1_load(a + 2 * g + 1);
            r = g1_add(p0, g1_mul_bits(g1_add(p1, g1_neg(p0)), x_bits));
        } else {
            r = g1_add(p0, g1_neg(g1_mul_bits(p0, x_bits)));
        }
        g1_store(out + g, r);
    }
}

// Sum of each of `rows` rows of `cols` points into d_out[rows] (device).
int g1_rowwise_sum_device(const G1Jac* d_a, size_t rows, size_t cols, G1Jac* d_out, Scratch& scratch, cudaStream_t s) {
    if (rows == 0) return ZKB_OK;
    if (rows > 65535) return fail(ZKB_ERR_LIMIT, "rowwise_sum: more than 65535 rows");
    if (cols == 0) {
        ZKB_LAUNCH(g1_fill_kernel, grid_for(rows, 128), 128, 0, s, d_out, G1Jac{}, rows);
        return ZKB_OK;
    }
    // stage 1: up to `parts` partial sums per row; stage 2: one block per row
    size_t parts = (cols + kSumThreads * 4 - 1) / (kSumThreads * 4);
    const size_t cap = ((size_t)sm_count() * 16 + rows - 1) / rows;
    if (parts > cap) parts = cap;
    if (parts < 1) parts = 1;
    if (parts == 1) {
        ZKB_LAUNCH(g1_row_partial_sum_kernel, dim3(1, (unsigned)rows), kSumThreads, 0, s, d_a, cols, d_out);
        return ZKB_OK;
    }
    G1Jac* part = scratch.get_n<G1Jac>(rows * parts);
    if (!part) return ZKB_ERR_CUDA;
    ZKB_LAUNCH(g1_row_partial_sum_kernel, dim3((unsigned)parts, (unsigned)rows), kSumThreads, 0, s, d_a, cols, part);
    ZKB_LAUNCH(g1_row_partial_sum_kernel, dim3(1, (unsigned)rows), kSumThreads, 0, s, part, parts, d_out);
    return ZKB_OK;
}

}  // namespace zkb

using namespace zkb;
#define G1(p) reinterpret_cast<G1Jac*>(p)
#define CG1(p) reinterpret_cast<const G1Jac*>(p)
#define CFR(p) reinterpret_cast<const Fr*>(p)

static inline G1Jac host_g1(const zkb_g1_t& h) {
    G1Jac r;
    memcpy(&r, &h, sizeof(G1Jac));
    return r;
}
static inline Fr host_fr(const zkb_fr_t& h) {
    Fr r;
    memcpy(r.v, h.val, 32);
    return r;
}

extern "C" {

int zkb_g1_fill(zkb_g1_t* d_out, const zkb_g1_t* h_val, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_fill_kernel, grid_for(n, 128), 128, 0, as_stream(stream), G1(d_out), host_g1(*h_val), n);
    return ZKB_OK;
}
int zkb_g1_neg(const zkb_g1_t* d_a, zkb_g1_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_neg_kernel, grid_for(n, 128), 128, 0, as_stream(stream), CG1(d_a), G1(d_out), n);
    return ZKB_OK;
}
int zkb_g1_add(const zkb_g1_t* d_a, const zkb_g1_t* d_b, zkb_g1_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_binary_kernel<G1Bin::Add>, grid_for(n, kG1Threads), kG1Threads, 0, as_stream(stream), CG1(d_a), CG1(d_b), G1(d_out), n);
    return ZKB_OK;
}
int zkb_g1_sub(const zkb_g1_t* d_a, const zkb_g1_t* d_b, zkb_g1_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_binary_kernel<G1Bin::Sub>, grid_for(n, kG1Threads), kG1Threads, 0, as_stream(stream), CG1(d_a), CG1(d_b), G1(d_out), n);
    return ZKB_OK;
}
int zkb_g1_add_scalar(const zkb_g1_t* d_a, const zkb_g1_t* h_x, zkb_g1_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_add_scalar_kernel, grid_for(n, kG1Threads), kG1Threads, 0, as_stream(stream), CG1(d_a), host_g1(*h_x), G1(d_out), n);
    return ZKB_OK;
}
int zkb_g1_from_affine(const zkb_g1_affine_t* d_a, zkb_g1_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_from_affine_kernel, grid_for(n, 128), 128, 0, as_stream(stream), reinterpret_cast<const G1Aff*>(d_a), G1(d_out), n);
    return ZKB_OK;
}
int zkb_g1_to_affine(const zkb_g1_t* d_a, zkb_g1_affine_t* d_out, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    ZKB_LAUNCH(g1_to_affine_kernel, grid_for(n, kG1Threads), kG1Threads, 0, as_stream(stream), CG1(d_a), reinterpret_cast<G1Aff*>(d_out), n);
    return ZKB_OK;
}
int zkb_g1_mul(const zkb_g1_t* d_g, size_t n_g, const zkb_fr_t* d_scalars, size_t n, zkb_g1_t* d_out, void* stream) {
    if (!n) return ZKB_OK;
    if (!n_g || n % n_g) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    ZKB_LAUNCH(g1_mul_kernel, grid_for(n, kG1Threads), kG1Threads, 0, as_stream(stream), CG1(d_g), n_g, CFR(d_scalars), n, G1(d_out));
    return ZKB_OK;
}
int zkb_g1_sum(const zkb_g1_t* d_a, size_t n, zkb_g1_t* h_out, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (n == 0) { memset(h_out, 0, sizeof(*h_out)); return ZKB_OK; }
    Scratch scratch(s);
    G1Jac* d_out = scratch.get_n<G1Jac>(1);
    if (!d_out) return ZKB_ERR_CUDA;
    ZKB_TRY(g1_rowwise_sum_device(CG1(d_a), 1, n, d_out, scratch, s));
    ZKB_CUDA(cudaMemcpyAsync(h_out, d_out, sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}
int zkb_g1_rowwise_sum(const zkb_g1_t* d_a, size_t rows, size_t cols, zkb_g1_t* d_out, void* stream) {
    cudaStream_t s = as_stream(stream);
    Scratch scratch(s);
    return g1_rowwise_sum_device(CG1(d_a), rows, cols, G1(d_out), scratch, s);
}
int zkb_g1_mle_eval(const zkb_g1_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k, zkb_g1_t* h_out, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (k > 32 || n == 0) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    if (k >= 1 && (n <= ((size_t)1 << (k - 1)) || n > ((size_t)1 << k))) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    if (k == 0 && n != 1) return fail(ZKB_ERR_DIM, "Incompatible dimensions");
    Scratch scratch(s);
    G1Jac* buf[2] = {scratch.get_n<G1Jac>((n + 1) / 2), scratch.get_n<G1Jac>((n + 3) / 4 + 1)};
    if (!buf[0] || !buf[1]) return ZKB_ERR_CUDA;
    const G1Jac* cur = CG1(d_a);
    size_t n_in = n;
    for (unsigned r = 0; r < k; ++r) {
        const size_t n_out = (n_in + 1) / 2;
        // the reference hands the challenge through an un-Montgomery step before
        // reading its bits (g1-tensor.cu:491)
        const zkb_fr_t xb = hfr::store(hfr::from_mont(hfr::load(h_u[r])));
        ZKB_LAUNCH(g1_me_step_kernel, grid_for(n_out, kG1Threads), kG1Threads, 0, s, cur, n_in, n_out, host_fr(xb), buf[r & 1]);
        cur = buf[r & 1];
        n_in = n_out;
    }
    ZKB_CUDA(cudaMemcpyAsync(h_out, cur, sizeof(G1Jac), cudaMemcpyDeviceToHost, s));
    ZKB_CUDA(cudaStreamSynchronize(s));
    return ZKB_OK;
}

}  // extern "C"
