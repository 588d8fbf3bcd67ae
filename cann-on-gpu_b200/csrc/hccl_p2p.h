// Interface between the Hccl* entry points (hccl.cpp) and the peer-memory all-gather (hccl_p2p.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

// The few communicator operations the set-up needs, bound by hccl.cpp to the NCCL copy in use (0 = success).
struct P2pNccl {
    int (*comm_count)(void *comm, int *n);
    int (*comm_rank)(void *comm, int *r);
    int (*all_gather_bytes)(void *comm, const void *send, void *recv, size_t bytes, cudaStream_t s);
    int (*all_reduce_min_int)(void *comm, int *buf, cudaStream_t s);
};

// What the decode kernel's gathering epilogue needs (same fields as aclnnB200DecodeGather).
struct P2pGatherTarget {
    void *peer[8];
    const unsigned long long *calls;
    unsigned int nranks, rank;
    unsigned long long buf_bytes;
};
// The communicator's receive windows (set up collectively at first use, outside stream capture).  false: not available.
bool p2p_gather_target(const P2pNccl &nccl, void *comm, cudaStream_t s, P2pGatherTarget *t);
// Enqueues the receiver: the other ranks' packets of this call -> gathered [nranks][elems_per_rank] 16-bit elements.
// 0 = enqueued, -1 = not applicable or launch error.
int p2p_unpack(const P2pNccl &nccl, void *comm, void *gathered, uint64_t elems_per_rank, cudaStream_t s);
// The all-reduce form: every rank's matmul has sent its fp32 partial result [elems] to every window; out [elems] 16-bit
// values = their sum (fp32 accumulation in rank order, rounded once).  0 = enqueued.
int p2p_reduce(const P2pNccl &nccl, void *comm, void *out, uint64_t elems, bool bf16, cudaStream_t s);
// Releases the communicator's window (before the communicator is destroyed).
void p2p_forget(void *comm);
// 0, or the code a poll for a peer's packet left when it gave up (0x500 + the peer's rank).
unsigned int p2p_status();
unsigned int p2p_test_poll_runs_out(unsigned long long wait_ns);

// Implemented in hccl.cpp (they need its NCCL binding); used by the gathering matmul of hccl_matmul.cpp.
extern "C" int hccl_gather_target(void *comm, void *stream, P2pGatherTarget *t);                       // 1 = available
extern "C" int hccl_gather_unpack(void *comm, void *gathered, uint64_t elems_per_rank, void *stream);  // 0 = enqueued
extern "C" int hccl_gather_reduce(void *comm, void *out, uint64_t elems, int bf16, void *stream);       // 0 = enqueued
