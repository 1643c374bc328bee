// Library plumbing: error text, device memory entry points, scratch pool.
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace zkb {

static thread_local std::string g_last_error;
std::atomic<unsigned long long> g_launches{0};

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return ZKB_ERR_CUDA;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

Scratch::~Scratch() {
    for (int i = 0; i < n_; ++i) cudaFreeAsync(blocks_[i], stream_);
}

void* Scratch::get(size_t bytes) {
    if (n_ >= kMax) {
        set_error("scratch: too many blocks in one call");
        return nullptr;
    }
    if (bytes == 0) bytes = 16;
    void* p = nullptr;
    cudaError_t e = cudaMallocAsync(&p, bytes, stream_);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaMallocAsync(scratch)");
        return nullptr;
    }
    blocks_[n_++] = p;
    return p;
}

}  // namespace zkb

using namespace zkb;

extern "C" {

const char* zkb_last_error(void) { return g_last_error.c_str(); }
int zkb_version(void) { return 100; }
unsigned long long zkb_launch_count(void) { return g_launches.load(); }

int zkb_malloc(void** d_ptr, size_t bytes) {
    if (!d_ptr) return fail(ZKB_ERR_ARG, "zkb_malloc: null out pointer");
    static bool pool_ready = false;
    if (!pool_ready) {
        // keep freed scratch blocks cached in the stream-ordered pool instead of
        // returning them to the driver at every synchronisation
        int dev = 0;
        cudaMemPool_t pool;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
            unsigned long long thresh = ~0ull;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh);
        }
        pool_ready = true;
    }
    ZKB_CUDA(cudaMalloc(d_ptr, bytes ? bytes : 16));
    return ZKB_OK;
}
int zkb_free(void* d_ptr) {
    ZKB_CUDA(cudaFree(d_ptr));
    return ZKB_OK;
}
int zkb_memcpy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream) {
    ZKB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    ZKB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return ZKB_OK;
}
int zkb_memcpy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream) {
    ZKB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    ZKB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return ZKB_OK;
}
int zkb_memcpy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream) {
    ZKB_CUDA(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return ZKB_OK;
}
int zkb_memset0(void* d_dst, size_t bytes, void* stream) {
    ZKB_CUDA(cudaMemsetAsync(d_dst, 0, bytes, as_stream(stream)));
    return ZKB_OK;
}
int zkb_sync(void* stream) {
    ZKB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return ZKB_OK;
}

}  // extern "C"
