// Integer-pipe micro-benchmarks used as the roofline denominator of the MSM
// kernels (which are bound by 32-bit multiply-add issue, not by memory).
#include "common.cuh"
#include "field.cuh"

namespace zkb {

// MODE 0: independent mad.lo.u32 chains (IMAD)
// MODE 1: independent mad.wide.u32 chains (IMAD.WIDE, 64-bit accumulate)
// MODE 2: mad.lo.cc / madc.hi.cc carry chains, the instruction mix of the field multiplier
template <int MODE>
__global__ void __launch_bounds__(256) imad_bench_kernel(unsigned iters, unsigned seed, unsigned* __restrict__ sink) {
    unsigned a = seed ^ threadIdx.x, b = seed * 2654435761u + blockIdx.x;
    if (MODE == 0) {
        unsigned acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = a + i;
        for (unsigned it = 0; it < iters; ++it) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = acc[i] * a + b;
        }
        unsigned r = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) r ^= acc[i];
        if (r == 0x12345678u) sink[0] = r;
    } else if (MODE == 1) {
        unsigned long long acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = a + i;
        for (unsigned it = 0; it < iters; ++it) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = (unsigned long long)(unsigned)acc[i] * a + acc[i];
        }
        unsigned long long r = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) r ^= acc[i];
        if (r == 0x12345678ull) sink[0] = (unsigned)r;
    } else {
        unsigned ev[8], od[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { ev[i] = a + i; od[i] = b + i; }
        for (unsigned it = 0; it < iters; ++it) {
            // two independent 8-instruction carry chains, as in one operand-limb step
            ptx_mad_lo_cc(ev[0], a, b);
            ptx_madc_hi_cc(ev[1], a, b);
            ptx_madc_lo_cc(ev[2], a, b);
            ptx_madc_hi_cc(ev[3], a, b);
            ptx_madc_lo_cc(ev[4], a, b);
            ptx_madc_hi_cc(ev[5], a, b);
            ptx_madc_lo_cc(ev[6], a, b);
            ptx_madc_hi_cc(ev[7], a, b);
            ptx_mad_lo_cc(od[0], b, a);
            ptx_madc_hi_cc(od[1], b, a);
            ptx_madc_lo_cc(od[2], b, a);
            ptx_madc_hi_cc(od[3], b, a);
            ptx_madc_lo_cc(od[4], b, a);
            ptx_madc_hi_cc(od[5], b, a);
            ptx_madc_lo_cc(od[6], b, a);
            ptx_madc_hi_cc(od[7], b, a);
        }
        unsigned r = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) r ^= ev[i] ^ od[i];
        if (r == 0x12345678u) sink[0] = r;
    }
}

}  // namespace zkb

using namespace zkb;

extern "C" int zkb_bench_imad(int mode, unsigned iters, double* h_gops, void* stream) {
    cudaStream_t s = as_stream(stream);
    if (mode < 0 || mode > 2 || !h_gops) return fail(ZKB_ERR_ARG, "zkb_bench_imad: bad arguments");
    unsigned* sink = nullptr;
    ZKB_CUDA(cudaMallocAsync(&sink, 16, s));
    const unsigned grid = (unsigned)sm_count() * 8, block = 256;
    cudaEvent_t e0, e1;
    ZKB_CUDA(cudaEventCreate(&e0));
    ZKB_CUDA(cudaEventCreate(&e1));
    float best = 1e30f;
    for (int rep = 0; rep < 4; ++rep) {
        ZKB_CUDA(cudaEventRecord(e0, s));
        if (mode == 0) ZKB_LAUNCH(imad_bench_kernel<0>, grid, block, 0, s, iters, 12345u + rep, sink);
        else if (mode == 1) ZKB_LAUNCH(imad_bench_kernel<1>, grid, block, 0, s, iters, 12345u + rep, sink);
        else ZKB_LAUNCH(imad_bench_kernel<2>, grid, block, 0, s, iters, 12345u + rep, sink);
        ZKB_CUDA(cudaEventRecord(e1, s));
        ZKB_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        ZKB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    ZKB_CUDA(cudaFreeAsync(sink, s));
    const double per_thread = (mode == 2 ? 16.0 : 8.0) * iters;
    *h_gops = per_thread * grid * block / (best * 1e-3) / 1e9;
    return ZKB_OK;
}
