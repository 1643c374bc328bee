// The process's NCCL communicator (comm.cu), as seen by the sharded provers.
#pragma once
#include "common.cuh"

namespace zkb {

int comm_world();   // 0 until zkb_comm_init has run
int comm_rank();
// d_recv[p * bytes .. (p+1) * bytes) = rank p's d_send, queued on `s`
int comm_allgather(const void* d_send, void* d_recv, size_t bytes, cudaStream_t s);

}  // namespace zkb
