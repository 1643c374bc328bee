// Element kernels of the Rescaling and zkSoftmax operators.
#include "frutil.cuh"

namespace zkb {

// rescaling_kernel (rescaling.cu:8-21): centred remainder and exact quotient.
__global__ void rescale_kernel(const Fr* __restrict__ in, long sf, Fr* __restrict__ out, Fr* __restrict__ rem, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const long hsf = sf >> 1;
        const long x = fr_to_i64(fr_load(in + i));
        const long t = (x + hsf) % sf;
        const long x_rem = (t < 0 ? t + sf : t) - hsf;
        const long x_res = (x - x_rem) / sf;
        fr_store(out + i, fr_from_i64(x_res));
        fr_store(rem + i, fr_from_i64(x_rem));
    }
}

// zkrelu_decomp_kernel (zkrelu.cu:9-30): the rescaled value split into sign,
// magnitude and centred remainder; res = max(rescaled, 0).
__global__ void relu_decomp_kernel(const Fr* __restrict__ in, long sf, Fr* __restrict__ sign, Fr* __restrict__ mag,
                                   Fr* __restrict__ rem, Fr* __restrict__ res, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const long hsf = sf >> 1;
        const long x = fr_to_i64(fr_load(in + i));
        const long t = (x + hsf) % sf;
        const long x_rem = (t < 0 ? t + sf : t) - hsf;
        const long x_res = (x - x_rem) / sf;
        const bool pos = x_res >= 0;
        fr_store(sign + i, fr_from_u64(pos ? 1ull : 0ull));
        fr_store(mag + i, fr_from_i64(pos ? x_res : -x_res));
        fr_store(rem + i, fr_from_i64(x_rem));
        fr_store(res + i, pos ? fr_from_i64(x_res) : fr_zero());
    }
}

// zksoftmax_calculate_table (zksoftmax.cu:4-16).  The expression is kept in the
// reference's form so that the double-precision result rounds identically.
__global__ void softmax_table_kernel(Fr* __restrict__ table, double theta_k, double scaling_factor_in, double d, double Bk, uint32_t bk) {
    const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x;
    if (x < bk) {
        const unsigned long result = static_cast<unsigned long>(exp(log(theta_k) - (Bk / (scaling_factor_in * sqrt(d))) * x) + 0.5);
        fr_store(table + x, fr_from_u64(result));
    }
}

// zksoftmax_shift (zksoftmax.cu:20-32).  The row sum of exp() is a
// left-to-right double-precision chain in the reference; one warp per row
// evaluates the exp() terms in parallel (32 columns at a time, staged in shared
// memory) and lane 0 adds them in column order, which gives the same rounding.
static constexpr int kShiftWarps = 4;
__global__ void __launch_bounds__(kShiftWarps * 32) softmax_shift_kernel(const Fr* __restrict__ A, Fr* __restrict__ shift,
                                                                          Fr* __restrict__ out, size_t rows, size_t cols,
                                                                          double scaling_factor_in, double d) {
    __shared__ double terms[kShiftWarps][32];
    __shared__ Fr shift_s[kShiftWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (size_t row = (size_t)blockIdx.x * kShiftWarps + warp; row < rows; row += (size_t)gridDim.x * kShiftWarps) {
        double temp = 0.0;
        for (size_t c0 = 0; c0 < cols; c0 += 32) {
            const size_t c = c0 + lane;
            if (c < cols)
                terms[warp][lane] = exp(static_cast<double>(fr_to_i64(fr_load(A + row * cols + c))) / (scaling_factor_in * sqrt(d)));
            __syncwarp();
            if (lane == 0) {
                const int lim = (cols - c0 < 32) ? (int)(cols - c0) : 32;
                for (int k = 0; k < lim; ++k) temp += terms[warp][k];
            }
            __syncwarp();
        }
        if (lane == 0) {
            double x = scaling_factor_in * sqrt(d) * log(temp);
            x = x * 1UL;
            const long v = (x >= 0) ? static_cast<long>(x + 0.5) : static_cast<long>(x - 0.5);
            const Fr sv = fr_from_i64(v);
            shift_s[warp] = sv;
            fr_store(shift + row, sv);
        }
        __syncwarp();
        const Fr sv = shift_s[warp];
        for (size_t c = lane; c < cols; c += 32)
            fr_store(out + row * cols + c, fr_sub(fr_load(A + row * cols + c), sv));
        __syncwarp();
    }
}

struct Radices { uint32_t bs[16]; };
// zksoftmax_decompose_kernel (zksoftmax.cu:95-109): only values whose negation
// fits 64 bits are decomposed; others leave their digit slots untouched.
__global__ void softmax_decompose_kernel(const Fr* __restrict__ X, Radices r, unsigned K, Fr* __restrict__ out, size_t N) {
    for (size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x; g < N; g += (size_t)gridDim.x * blockDim.x) {
        const Fr mx = fr_neg(fr_load(X + g));
        if (fr_fits_u64(mx)) {
            unsigned long tmp = ((unsigned long)mx.v[1] << 32) | mx.v[0];
            for (unsigned i = 0; i < K; ++i) {
                fr_store(out + (size_t)i * N + g, fr_from_u64(tmp % r.bs[i]));
                tmp /= r.bs[i];
            }
        }
    }
}

}  // namespace zkb

using namespace zkb;

extern "C" {

int zkb_rescale(const zkb_fr_t* d_in, uint64_t scaling_factor, zkb_fr_t* d_out, zkb_fr_t* d_rem, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    if (scaling_factor == 0) return fail(ZKB_ERR_ARG, "Rescaling: scaling factor is zero");
    ZKB_LAUNCH(rescale_kernel, grid_for(n, 256), 256, 0, as_stream(stream), reinterpret_cast<const Fr*>(d_in),
               (long)scaling_factor, reinterpret_cast<Fr*>(d_out), reinterpret_cast<Fr*>(d_rem), n);
    return ZKB_OK;
}
int zkb_relu_decomp(const zkb_fr_t* d_in, uint64_t scaling_factor, zkb_fr_t* d_sign, zkb_fr_t* d_abs, zkb_fr_t* d_rem,
                    zkb_fr_t* d_res, size_t n, void* stream) {
    if (!n) return ZKB_OK;
    if (scaling_factor == 0) return fail(ZKB_ERR_ARG, "zkReLU: scaling factor is zero");
    ZKB_LAUNCH(relu_decomp_kernel, grid_for(n, 256), 256, 0, as_stream(stream), reinterpret_cast<const Fr*>(d_in),
               (long)scaling_factor, reinterpret_cast<Fr*>(d_sign), reinterpret_cast<Fr*>(d_abs), reinterpret_cast<Fr*>(d_rem),
               reinterpret_cast<Fr*>(d_res), n);
    return ZKB_OK;
}
int zkb_softmax_table(double theta_k, double scaling_factor_in, double d, double Bk, uint32_t bk, zkb_fr_t* d_table, void* stream) {
    if (!bk) return ZKB_OK;
    ZKB_LAUNCH(softmax_table_kernel, div_up(bk, 256), 256, 0, as_stream(stream), reinterpret_cast<Fr*>(d_table),
               theta_k, scaling_factor_in, d, Bk, bk);
    return ZKB_OK;
}
int zkb_softmax_shift(const zkb_fr_t* d_A, zkb_fr_t* d_shift, zkb_fr_t* d_out, size_t rows, size_t cols,
                      double scaling_factor_in, double d, void* stream) {
    if (!rows) return ZKB_OK;
    ZKB_LAUNCH(softmax_shift_kernel, grid_for(rows, kShiftWarps, 8), kShiftWarps * 32, 0, as_stream(stream),
               reinterpret_cast<const Fr*>(d_A), reinterpret_cast<Fr*>(d_shift), reinterpret_cast<Fr*>(d_out),
               rows, cols, scaling_factor_in, d);
    return ZKB_OK;
}
int zkb_softmax_decompose(const zkb_fr_t* d_X, const uint32_t* h_bs, unsigned K, zkb_fr_t* d_out, size_t N, void* stream) {
    if (!N || !K) return ZKB_OK;
    if (K > 16) return fail(ZKB_ERR_LIMIT, "zkSoftmax: more than 16 segments");
    Radices r;
    for (unsigned i = 0; i < 16; ++i) r.bs[i] = i < K ? h_bs[i] : 1u;
    for (unsigned i = 0; i < K; ++i)
        if (!h_bs[i]) return fail(ZKB_ERR_ARG, "zkSoftmax: zero radix");
    ZKB_LAUNCH(softmax_decompose_kernel, grid_for(N, 256), 256, 0, as_stream(stream), reinterpret_cast<const Fr*>(d_X), r, K,
               reinterpret_cast<Fr*>(d_out), N);
    return ZKB_OK;
}

}  // extern "C"
