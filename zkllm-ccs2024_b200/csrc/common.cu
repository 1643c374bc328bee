// Library plumbing: error text, device memory entry points, scratch pool.
#include "common.cuh"

#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <map>
#include <mutex>
#include <vector>

namespace zkb {

static thread_local std::string g_last_error;
std::atomic<unsigned long long> g_launches{0};
std::atomic<cudaStream_t> g_default_stream{nullptr};

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return ZKB_ERR_CUDA;
}

// ---- per-kernel timing ------------------------------------------------------------
bool g_profile_on = false;
namespace {
struct ProfRec { std::string name; cudaEvent_t e0, e1; };
std::vector<ProfRec> g_prof;
std::mutex g_prof_mu;
}  // namespace

void profile_begin(const char* name, cudaStream_t s) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    ProfRec r;
    r.name = name;
    r.e0 = r.e1 = nullptr;
    if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) {
        // keep begin/end paired: a record without events is skipped by profile_end and the reader
        if (r.e0) cudaEventDestroy(r.e0);
        r.e0 = r.e1 = nullptr;
        g_prof.push_back(r);
        return;
    }
    cudaEventRecord(r.e0, s);
    g_prof.push_back(r);
}
void profile_end(cudaStream_t s) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    if (!g_prof.empty() && g_prof.back().e1) cudaEventRecord(g_prof.back().e1, s);
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

static bool nvtx_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("ZKLLM_NVTX");
        return e && e[0] == '1';
    }();
    return on;
}
ApiRange::ApiRange(const char* name) : on(nvtx_enabled()) {
    if (on) nvtxRangePushA(name);
}
ApiRange::~ApiRange() {
    if (on) nvtxRangePop();
}

SideStream* side_stream() {
    static SideStream table[64];
    static bool made[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { fail(ZKB_ERR_CUDA, "side stream: no current device"); return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    if (!made[dev]) {
        SideStream& t = table[dev];
        if (cudaStreamCreateWithFlags(&t.st, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&t.join, cudaEventDisableTiming) != cudaSuccess) {
            fail(ZKB_ERR_CUDA, "side stream: cannot create stream or events");
            return nullptr;
        }
        made[dev] = true;
    }
    return &table[dev];
}

// The library's own stream-ordered memory pool, one per device, created on first use.  Its release
// threshold is unlimited, so freed blocks stay cached (with the default threshold of 0 a pool hands
// its memory back to the driver at every synchronisation and the next call pays for mapping it again);
// zkb_pool_trim gives cached memory back.  The device's default pool, which other users of
// cudaMallocAsync in the same process share, is left as it is.
static cudaMemPool_t library_pool() {
    static cudaMemPool_t pools[64];
    static bool made[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!made[dev]) {
        cudaMemPoolProps props;
        memset(&props, 0, sizeof(props));
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        unsigned long long thresh = ~0ull;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh);
        pools[dev] = pool;
        made[dev] = true;
    }
    return pools[dev];
}
static cudaError_t pool_alloc(void** p, size_t bytes, cudaStream_t s) {
    cudaMemPool_t pool = library_pool();
    return pool ? cudaMallocFromPoolAsync(p, bytes, pool, s) : cudaMallocAsync(p, bytes, s);
}

// Host time spent inside the allocator calls, reported by zkb_profile_read as
// "host:<what>" lines next to the kernels (only while profiling is enabled).
static std::atomic<unsigned long long> g_alloc_ns[3], g_alloc_calls[3];
static const char* const kAllocNames[3] = {"host:scratch_alloc", "host:zkb_malloc", "host:zkb_free"};
struct AllocClock {
    int which;
    std::chrono::steady_clock::time_point t0;
    explicit AllocClock(int w) : which(w) { if (g_profile_on) t0 = std::chrono::steady_clock::now(); }
    ~AllocClock() {
        if (!g_profile_on) return;
        g_alloc_ns[which] += (unsigned long long)std::chrono::duration_cast<std::chrono::nanoseconds>(
                                 std::chrono::steady_clock::now() - t0).count();
        g_alloc_calls[which] += 1;
    }
};

// ---- guard bands (debug aid; stands in for a memory checker) ---------------------------
// With ZKLLM_GUARD=1 in the environment, or after zkb_guard_enable(1), every block the library hands out - the
// scratch blocks of all entry points and the buffers of zkb_malloc - is allocated with 256 bytes before and after it
// that hold a fixed pattern.  When the block is released a small kernel compares the bands with the pattern, in the
// stream's order, and counts a block whose band was written: a kernel that stores outside its buffer by up to 64
// words is caught wherever the buffer came from the library.  zkb_guard_report returns the counts.  Reads outside
// a buffer are not seen (the bands are valid memory); wrong results from them are what the parity tests catch.
constexpr size_t kGuardBytes = 256;
constexpr uint32_t kGuardWord = 0xA5C3F00Du;
struct GuardStats { unsigned long long blocks, damaged, first_bytes; unsigned first_side, pad; };
__device__ GuardStats g_guard_stats;
static std::atomic<int> g_guard_on{-1};          // -1: not decided yet (environment), 0 / 1

static bool guard_on() {
    int v = g_guard_on.load();
    if (v < 0) {
        const char* e = std::getenv("ZKLLM_GUARD");
        v = (e && e[0] == '1') ? 1 : 0;
        g_guard_on.store(v);
    }
    return v == 1;
}
static size_t guard_round(size_t bytes) { return (bytes + 3) & ~(size_t)3; }

__global__ void guard_fill_kernel(uint32_t* lo, uint32_t* hi) {
    lo[threadIdx.x] = kGuardWord;
    hi[threadIdx.x] = kGuardWord;
}
__global__ void guard_check_kernel(const uint32_t* lo, const uint32_t* hi, unsigned long long bytes) {
    const bool bad_lo = lo[threadIdx.x] != kGuardWord, bad_hi = hi[threadIdx.x] != kGuardWord;
    const int any = __syncthreads_or(bad_lo || bad_hi);
    const int any_lo = __syncthreads_or(bad_lo);
    if (threadIdx.x == 0) {
        atomicAdd(&g_guard_stats.blocks, 1ull);
        if (any && atomicAdd(&g_guard_stats.damaged, 1ull) == 0) {
            g_guard_stats.first_bytes = bytes;
            g_guard_stats.first_side = any_lo ? 0u : 1u;
        }
    }
}
// base: what the pool returned for bytes + 2 bands; returns the user pointer
static void* guard_arm(void* base, size_t bytes, cudaStream_t s) {
    char* b = static_cast<char*>(base);
    guard_fill_kernel<<<1, kGuardBytes / 4, 0, s>>>(reinterpret_cast<uint32_t*>(b),
                                                    reinterpret_cast<uint32_t*>(b + kGuardBytes + guard_round(bytes)));
    return b + kGuardBytes;
}
static void guard_verify(void* base, size_t bytes, cudaStream_t s) {
    char* b = static_cast<char*>(base);
    guard_check_kernel<<<1, kGuardBytes / 4, 0, s>>>(reinterpret_cast<const uint32_t*>(b),
                                                     reinterpret_cast<const uint32_t*>(b + kGuardBytes + guard_round(bytes)),
                                                     (unsigned long long)bytes);
}
// buffers of zkb_malloc that carry bands: user pointer -> user bytes
static std::mutex g_guard_mu;
static std::map<void*, size_t> g_guarded;

Scratch::~Scratch() {
    for (int i = 0; i < n_; ++i) {
        if (guarded_[i]) guard_verify(blocks_[i], guarded_[i], stream_);
        cudaFreeAsync(blocks_[i], stream_);
    }
}

void* Scratch::get(size_t bytes) {
    if (n_ >= kMax) {
        set_error("scratch: too many blocks in one call");
        return nullptr;
    }
    if (bytes == 0) bytes = 16;
    AllocClock clock(0);
    const bool guard = guard_on();
    void* p = nullptr;
    cudaError_t e = pool_alloc(&p, guard ? guard_round(bytes) + 2 * kGuardBytes : bytes, stream_);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaMallocAsync(scratch)");
        return nullptr;
    }
    blocks_[n_] = p;
    guarded_[n_] = guard ? bytes : 0;
    ++n_;
    return guard ? guard_arm(p, bytes, stream_) : p;
}

}  // namespace zkb

using namespace zkb;

extern "C" {

const char* zkb_last_error(void) { return g_last_error.c_str(); }
int zkb_version(void) { return 100; }
unsigned long long zkb_launch_count(void) { return g_launches.load(); }

int zkb_profile_enable(int on) {
    g_profile_on = on != 0;
    return ZKB_OK;
}
int zkb_profile_reset(void) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    for (auto& r : g_prof) { if (r.e0) cudaEventDestroy(r.e0); if (r.e1) cudaEventDestroy(r.e1); }
    g_prof.clear();
    for (int i = 0; i < 3; ++i) { g_alloc_ns[i] = 0; g_alloc_calls[i] = 0; }
    return ZKB_OK;
}
int zkb_profile_read(char* buf, size_t cap) {
    if (!buf || cap == 0) return fail(ZKB_ERR_ARG, "zkb_profile_read: no buffer");
    ZKB_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lk(g_prof_mu);
    std::map<std::string, std::pair<unsigned long long, double>> agg;
    for (auto& r : g_prof) {
        float ms = 0.f;
        if (r.e0 && r.e1 && cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) {
            auto& a = agg[r.name];
            a.first += 1;
            a.second += ms;
        }
    }
    std::string out;
    for (auto& kv : agg) {
        char line[256];
        snprintf(line, sizeof(line), "%s,%llu,%.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        out += line;
    }
    for (int i = 0; i < 3; ++i) {
        if (!g_alloc_calls[i]) continue;
        char line[256];
        snprintf(line, sizeof(line), "%s,%llu,%.6f\n", kAllocNames[i], (unsigned long long)g_alloc_calls[i], g_alloc_ns[i] * 1e-6);
        out += line;
    }
    if (out.size() + 1 > cap) return fail(ZKB_ERR_LIMIT, "zkb_profile_read: buffer too small");
    memcpy(buf, out.c_str(), out.size() + 1);
    return ZKB_OK;
}

// Device buffers come from the library's stream-ordered pool (which keeps freed
// memory for reuse), allocated and released on the null stream.  zkb_malloc
// returns memory that is usable at once on any stream; zkb_free first waits for
// the whole device, like cudaFree, so work still running on any stream is safe.
int zkb_malloc(void** d_ptr, size_t bytes) {
    if (!d_ptr) return fail(ZKB_ERR_ARG, "zkb_malloc: null out pointer");
    AllocClock clock(1);
    if (!bytes) bytes = 16;
    if (guard_on()) {
        void* base = nullptr;
        ZKB_CUDA(pool_alloc(&base, guard_round(bytes) + 2 * kGuardBytes, as_stream(nullptr)));
        *d_ptr = guard_arm(base, bytes, as_stream(nullptr));
        std::lock_guard<std::mutex> lk(g_guard_mu);
        g_guarded[*d_ptr] = bytes;
    } else {
        ZKB_CUDA(pool_alloc(d_ptr, bytes, as_stream(nullptr)));
    }
    ZKB_CUDA(cudaStreamSynchronize(as_stream(nullptr)));
    return ZKB_OK;
}
static int free_after(void* d_ptr, bool whole_device);
int zkb_free(void* d_ptr) { return free_after(d_ptr, true); }
int zkb_free_default_stream(void* d_ptr) { return free_after(d_ptr, false); }
static int free_after(void* d_ptr, bool whole_device) {
    if (!d_ptr) return ZKB_OK;
    AllocClock clock(2);
    if (whole_device) ZKB_CUDA(cudaDeviceSynchronize());
    else ZKB_CUDA(cudaStreamSynchronize(as_stream(nullptr)));
    size_t guarded = 0;
    {
        std::lock_guard<std::mutex> lk(g_guard_mu);
        auto it = g_guarded.find(d_ptr);
        if (it != g_guarded.end()) { guarded = it->second; g_guarded.erase(it); }
    }
    if (guarded) {
        void* base = static_cast<char*>(d_ptr) - kGuardBytes;
        guard_verify(base, guarded, as_stream(nullptr));
        ZKB_CUDA(cudaFreeAsync(base, as_stream(nullptr)));
        return ZKB_OK;
    }
    ZKB_CUDA(cudaFreeAsync(d_ptr, as_stream(nullptr)));
    return ZKB_OK;
}
int zkb_set_default_stream(void* stream) {
    g_default_stream.store(reinterpret_cast<cudaStream_t>(stream));
    return ZKB_OK;
}
int zkb_stream_create(int high_priority, void** stream) {
    if (!stream) return fail(ZKB_ERR_ARG, "zkb_stream_create: null out pointer");
    int least = 0, greatest = 0;
    ZKB_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    cudaStream_t st = nullptr;
    ZKB_CUDA(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, high_priority ? greatest : least));
    *stream = st;
    return ZKB_OK;
}
int zkb_stream_destroy(void* stream) {
    if (!stream) return ZKB_OK;
    if (g_default_stream.load() == reinterpret_cast<cudaStream_t>(stream)) g_default_stream.store(nullptr);
    ZKB_CUDA(cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream)));
    return ZKB_OK;
}
int zkb_guard_enable(int on) {
    g_guard_on.store(on ? 1 : 0);
    return ZKB_OK;
}
int zkb_guard_report(unsigned long long* blocks_checked, unsigned long long* blocks_damaged,
                     unsigned long long* first_damaged_bytes, int* first_damaged_side, int reset) {
    ZKB_CUDA(cudaDeviceSynchronize());
    GuardStats st;
    ZKB_CUDA(cudaMemcpyFromSymbol(&st, g_guard_stats, sizeof(st)));
    if (blocks_checked) *blocks_checked = st.blocks;
    if (blocks_damaged) *blocks_damaged = st.damaged;
    if (first_damaged_bytes) *first_damaged_bytes = st.first_bytes;
    if (first_damaged_side) *first_damaged_side = st.damaged ? (int)st.first_side : -1;
    if (reset) {
        memset(&st, 0, sizeof(st));
        ZKB_CUDA(cudaMemcpyToSymbol(g_guard_stats, &st, sizeof(st)));
    }
    return ZKB_OK;
}
int zkb_pool_trim(size_t keep_bytes) {
    cudaMemPool_t pool = library_pool();
    if (!pool) return ZKB_OK;
    ZKB_CUDA(cudaDeviceSynchronize());
    ZKB_CUDA(cudaMemPoolTrimTo(pool, keep_bytes));
    return ZKB_OK;
}
int zkb_host_alloc(void** h_ptr, size_t bytes) {
    if (!h_ptr) return fail(ZKB_ERR_ARG, "zkb_host_alloc: null out pointer");
    ZKB_CUDA(cudaHostAlloc(h_ptr, bytes ? bytes : 16, cudaHostAllocDefault));
    return ZKB_OK;
}
int zkb_host_free(void* h_ptr) {
    if (!h_ptr) return ZKB_OK;
    ZKB_CUDA(cudaFreeHost(h_ptr));
    return ZKB_OK;
}
int zkb_memcpy_h2d_async(void* d_dst, const void* h_src, size_t bytes, void* stream) {
    ZKB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return ZKB_OK;
}
int zkb_memcpy_d2h_async(void* h_dst, const void* d_src, size_t bytes, void* stream) {
    ZKB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
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
