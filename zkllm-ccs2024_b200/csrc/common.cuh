// Shared host-side plumbing for the C-ABI translation units: status codes,
// error text, launch checking and the stream-ordered scratch pool.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <atomic>
#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/zkllm_b200.h"

namespace zkb {

// Thread-local text of the last failure, returned by zkb_last_error().
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

#define ZKB_CUDA(call)                                                    \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) return ::zkb::cuda_fail(e__, #call);      \
    } while (0)

#define ZKB_LAUNCH_CHECK(name)                                            \
    do {                                                                  \
        cudaError_t e__ = cudaGetLastError();                             \
        if (e__ != cudaSuccess) return ::zkb::cuda_fail(e__, name);       \
    } while (0)

#define ZKB_TRY(expr)                                                     \
    do {                                                                  \
        int rc__ = (expr);                                                \
        if (rc__ != ZKB_OK) return rc__;                                  \
    } while (0)

// Count of kernels launched by this library in this process (zkb_launch_count()).
extern std::atomic<unsigned long long> g_launches;

// Optional per-kernel timing (zkb_profile_*): when enabled every launch is
// bracketed by two events on its stream.
extern bool g_profile_on;
void profile_begin(const char* name, cudaStream_t s);
void profile_end(cudaStream_t s);

// Launch + count + check.  Usage: ZKB_LAUNCH(kernel, grid, block, smem, stream, args...)
#define ZKB_LAUNCH(kernel, grid, block, smem, stream, ...)                \
    do {                                                                  \
        if (::zkb::g_profile_on) ::zkb::profile_begin(#kernel, (stream)); \
        kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);       \
        if (::zkb::g_profile_on) ::zkb::profile_end((stream));            \
        ::zkb::g_launches.fetch_add(1, std::memory_order_relaxed);        \
        ZKB_LAUNCH_CHECK(#kernel);                                        \
    } while (0)

// A named range around an entry point for timeline tools (NVTX push/pop), active only when the
// environment variable ZKLLM_NVTX is 1 at the first call; otherwise one branch.
struct ApiRange {
    bool on;
    explicit ApiRange(const char* name);
    ~ApiRange();
};
#define ZKB_API_RANGE() ::zkb::ApiRange api_range__(__func__)

// A null stream argument of the C ABI means the CUDA default stream, unless the host named a stream of its own for
// that role (zkb_set_default_stream): e.g. a high-priority stream, so that its short kernels are scheduled ahead of
// the long-running blocks of openings in flight on the library's own streams.
extern std::atomic<cudaStream_t> g_default_stream;
inline cudaStream_t as_stream(void* s) {
    return s ? reinterpret_cast<cudaStream_t>(s) : g_default_stream.load(std::memory_order_relaxed);
}

// Number of SMs of the current device (cached per device).
int sm_count();

// Scratch memory that lives for one entry-point call.  Blocks come from the
// library's stream-ordered pool (cudaMallocFromPoolAsync), so a call neither blocks the
// device nor pays a cudaMalloc; every block is released in the destructor in
// stream order.
class Scratch {
public:
    explicit Scratch(cudaStream_t s) : stream_(s) {}
    ~Scratch();
    Scratch(const Scratch&) = delete;
    Scratch& operator=(const Scratch&) = delete;
    // returns nullptr and records the error on failure
    void* get(size_t bytes);
    template <class T> T* get_n(size_t n) { return static_cast<T*>(get(n * sizeof(T))); }
private:
    static constexpr int kMax = 256;
    cudaStream_t stream_;
    void* blocks_[kMax];        // what the pool returned
    size_t guarded_[kMax];      // user bytes of a block with guard bands, 0 for a plain block
    int n_ = 0;
};

// A second stream per device for work that may run beside the caller's stream,
// with the two events that fork from and join back into it.  Created on first use.
// `busy` is held for the length of a call that uses the stream, so two host threads
// on one device take turns.  Drain waits for the stream when a call leaves early.
// Memory that work on the side stream touches is allocated from a Scratch bound to
// that stream (stream-ordered allocations are only ordered on their own stream).
struct SideStream { cudaStream_t st; cudaEvent_t fork, join; std::mutex busy; };
struct Drain {
    cudaStream_t st;
    ~Drain() { cudaStreamSynchronize(st); }
};
SideStream* side_stream();   // nullptr (and the error text set) on failure

inline unsigned div_up(size_t a, size_t b) { return (unsigned)((a + b - 1) / b); }

// Host: round polynomials of the lookup sumcheck from its per-round sums, with the
// reference's checks (defined in combine.cu; used by the single- and the multi-GPU prover).
int tlookup_assemble(const zkb_fr_t* sums, size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_u,
                     const zkb_fr_t* h_v, zkb_fr_t* h_polys, zkb_fr_t* h_final);
// The verifier equations of multi_hadamard_sumchecks (proof.cu:190-241) on the K + 1 coefficients of each of the kN
// rounds: claim == (c * eq(u))(0) + (c * eq(u))(1), next claim = c(v).  Host arithmetic (combine.cu).
int hadamard_replay(const zkb_fr_t* h_claim, const zkb_fr_t* h_polys, unsigned K, unsigned kN, const zkb_fr_t* h_u,
                    const zkb_fr_t* h_v, zkb_fr_t* h_final);

}  // namespace zkb
