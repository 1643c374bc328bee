// The exchange step of the multi-GPU provers: one process per GPU, one NCCL
// communicator per process, plain ncclAllGather on this GPU's own buffers.
//
// The reference is single-GPU, so nothing here replaces a reference function.  The
// sharded provers (zkb_commit_i32_sharded, zkb_zkfc_prove_sharded,
// zkb_tlookup_prove_sharded) run all their local work first and exchange ONCE: a few
// hundred bytes of partial sums, or the m / P row commitments of a rank.  Modular
// sums and G1 sums are not reductions NCCL offers, so every exchange is an
// all-gather and the sums are formed after it.
//
// NCCL is loaded at run time (dlopen): a single-GPU process never needs it, and a
// process that already holds a copy (one loaded by PyTorch, say) shares that copy
// instead of bringing a second one.
#include "comm.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace zkb {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_api;
ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 0;
std::mutex g_mu;

int load_api() {
    if (g_api.handle) return ZKB_OK;
    // A copy the process already has comes first: two NCCL builds under the same library name cannot
    // live in one process, so a host that will load its own NCCL later (PyTorch, say) must do so before
    // this call, or name that copy in ZKLLM_NCCL_LIB.
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) {
        const char* named = std::getenv("ZKLLM_NCCL_LIB");
        if (named && named[0]) h = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
    }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(ZKB_ERR_ARG, std::string("comm: cannot load NCCL: ") + dlerror());
    NcclApi a;
    a.handle = h;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    if (!a.GetUniqueId || !a.CommInitRank || !a.AllGather || !a.CommDestroy || !a.GetErrorString)
        return fail(ZKB_ERR_ARG, "comm: the NCCL library lacks a required entry point");
    g_api = a;
    return ZKB_OK;
}

int nccl_fail(ncclResult_t r, const char* what) {
    return fail(ZKB_ERR_CUDA, std::string(what) + ": " + (g_api.GetErrorString ? g_api.GetErrorString(r) : "NCCL error"));
}

}  // namespace

int comm_world() { return g_world; }
int comm_rank() { return g_rank; }

int comm_allgather(const void* d_send, void* d_recv, size_t bytes, cudaStream_t s) {
    if (!g_comm) return fail(ZKB_ERR_ARG, "comm: not initialised (zkb_comm_init)");
    if (bytes == 0) return ZKB_OK;
    const ncclResult_t r = g_api.AllGather(d_send, d_recv, bytes, ncclChar, g_comm, s);
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllGather");
    return ZKB_OK;
}

}  // namespace zkb

using namespace zkb;

extern "C" {

int zkb_comm_unique_id(unsigned char* id128) {
    if (!id128) return fail(ZKB_ERR_ARG, "comm: null id buffer");
    std::lock_guard<std::mutex> lk(g_mu);
    ZKB_TRY(load_api());
    static_assert(sizeof(ncclUniqueId) == 128, "the id buffer of the C ABI is 128 bytes");
    ncclUniqueId id;
    const ncclResult_t r = g_api.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id128, &id, sizeof(id));
    return ZKB_OK;
}

int zkb_comm_init(int rank, int world, const unsigned char* id128) {
    if (!id128 || world < 1 || rank < 0 || rank >= world) return fail(ZKB_ERR_ARG, "comm: bad rank, world or id");
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_comm) return fail(ZKB_ERR_ARG, "comm: already initialised");
    ZKB_TRY(load_api());
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    const ncclResult_t r = g_api.CommInitRank(&c, world, id, rank);   // on the current device
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
    g_comm = c;
    g_rank = rank;
    g_world = world;
    return ZKB_OK;
}

int zkb_comm_info(int* rank, int* world) {
    if (rank) *rank = g_rank;
    if (world) *world = g_world;
    return ZKB_OK;
}

int zkb_comm_destroy(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_comm) return ZKB_OK;
    const ncclResult_t r = g_api.CommDestroy(g_comm);
    g_comm = nullptr;
    g_world = 0;
    g_rank = 0;
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommDestroy");
    return ZKB_OK;
}

int zkb_comm_allgather(const void* d_send, void* d_recv, size_t bytes_per_rank, void* stream) {
    return comm_allgather(d_send, d_recv, bytes_per_rank, as_stream(stream));
}

}  // extern "C"
