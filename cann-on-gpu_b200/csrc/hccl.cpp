// Hccl* collectives over NCCL, for gathering column-sharded matmul outputs across the GPUs of a
// box (NVLink 5 / NVSwitch).  Same contract as the reference's cuda/src/hccl.cu:47-172: the root
// info blob carries the NCCL unique id, one NCCL communicator per HcclComm, every collective is
// enqueued on the caller's stream.
//
// NCCL is bound at first use, not at load time: a process that already holds an NCCL (for example
// the one bundled with PyTorch) keeps using that copy, and merely loading this library pulls no
// second NCCL into the process.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>

#include "hccl/hccl.h"
#include "hccl_p2p.h"

namespace {
static_assert(sizeof(ncclUniqueId) <= HCCL_ROOT_INFO_BYTES, "root info must hold the NCCL unique id");

struct Nccl {
    decltype(&::ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&::ncclCommInitRank) CommInitRank = nullptr;
    decltype(&::ncclCommDestroy) CommDestroy = nullptr;
    decltype(&::ncclAllReduce) AllReduce = nullptr;
    decltype(&::ncclAllGather) AllGather = nullptr;
    decltype(&::ncclReduceScatter) ReduceScatter = nullptr;
    decltype(&::ncclBroadcast) Broadcast = nullptr;
    decltype(&::ncclCommCount) CommCount = nullptr;
    decltype(&::ncclCommUserRank) CommUserRank = nullptr;
    bool ok = false;
};

const Nccl &nccl() {
    static Nccl n = [] {
        Nccl t;
        void *h = nullptr;
        // B200_HCCL_NCCL_LIB names the library to bind instead (the tests hand in a stand-in whose rendezvous
        // never completes, to exercise the bootstrap time limit without a GPU)
        if (const char *over = getenv("B200_HCCL_NCCL_LIB")) h = dlopen(over, RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // a copy the process already holds
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            fprintf(stderr, "[b200-hccl] NCCL not found: %s\n", dlerror());
            return t;
        }
#define BIND(name) t.name = reinterpret_cast<decltype(t.name)>(dlsym(h, "nccl" #name))
        BIND(GetUniqueId); BIND(CommInitRank); BIND(CommDestroy); BIND(AllReduce); BIND(AllGather);
        BIND(ReduceScatter); BIND(Broadcast); BIND(CommCount); BIND(CommUserRank);
#undef BIND
        t.ok = t.GetUniqueId && t.CommInitRank && t.CommDestroy && t.AllReduce && t.AllGather && t.ReduceScatter &&
               t.Broadcast && t.CommCount && t.CommUserRank;
        return t;
    }();
    return n;
}
#define NEED_NCCL() do { if (!nccl().ok) return HCCL_E_UNAVAIL; } while (0)

bool to_nccl(HcclDataType t, ncclDataType_t *o) {
    switch (t) {
        case HCCL_DATA_TYPE_INT8: *o = ncclInt8; return true;
        case HCCL_DATA_TYPE_UINT8: *o = ncclUint8; return true;
        case HCCL_DATA_TYPE_INT32: *o = ncclInt32; return true;
        case HCCL_DATA_TYPE_UINT32: *o = ncclUint32; return true;
        case HCCL_DATA_TYPE_INT64: *o = ncclInt64; return true;
        case HCCL_DATA_TYPE_UINT64: *o = ncclUint64; return true;
        case HCCL_DATA_TYPE_FP16: *o = ncclFloat16; return true;
        case HCCL_DATA_TYPE_FP32: *o = ncclFloat32; return true;
        case HCCL_DATA_TYPE_FP64: *o = ncclFloat64; return true;
        case HCCL_DATA_TYPE_BFP16: *o = ncclBfloat16; return true;
        default: return false;
    }
}
bool to_nccl(HcclReduceOp op, ncclRedOp_t *o) {
    switch (op) {
        case HCCL_REDUCE_SUM: *o = ncclSum; return true;
        case HCCL_REDUCE_PROD: *o = ncclProd; return true;
        case HCCL_REDUCE_MAX: *o = ncclMax; return true;
        case HCCL_REDUCE_MIN: *o = ncclMin; return true;
    }
    return false;
}
// what the peer-memory all-gather needs of the communicator
const P2pNccl &p2p_table() {
    static const P2pNccl t = {
        [](void *c, int *n) { return (int)nccl().CommCount((ncclComm_t)c, n); },
        [](void *c, int *r) { return (int)nccl().CommUserRank((ncclComm_t)c, r); },
        [](void *c, const void *send, void *recv, size_t bytes, cudaStream_t s) {
            return (int)nccl().AllGather(send, recv, bytes, ncclInt8, (ncclComm_t)c, s);
        },
        [](void *c, int *buf, cudaStream_t s) { return (int)nccl().AllReduce(buf, buf, 1, ncclInt32, ncclMin, (ncclComm_t)c, s); },
    };
    return t;
}
HcclResult from_nccl(ncclResult_t r) {
    switch (r) {
        case ncclSuccess: return HCCL_SUCCESS;
        case ncclInvalidArgument: case ncclInvalidUsage: return HCCL_E_PARA;
        case ncclSystemError: case ncclRemoteError: return HCCL_E_NETWORK;
        default: return HCCL_E_INTERNAL;
    }
}
}  // namespace

extern "C" {

HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo) {
    NEED_NCCL();
    if (!rootInfo) return HCCL_E_PTR;
    ncclUniqueId id;
    ncclResult_t r = nccl().GetUniqueId(&id);
    if (r != ncclSuccess) return from_nccl(r);
    memset(rootInfo->internal, 0, sizeof(rootInfo->internal));
    memcpy(rootInfo->internal, &id, sizeof(id));
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm) {
    NEED_NCCL();
    if (!rootInfo || !comm) return HCCL_E_PTR;
    if (nRanks == 0 || rank >= nRanks) return HCCL_E_PARA;
    ncclUniqueId id;
    memcpy(&id, rootInfo->internal, sizeof(id));
    // The rendezvous blocks until every rank has joined.  A rank that never joins (it died, or was never started)
    // would hold the others forever, so the call runs on a helper thread and is given up after
    // B200_HCCL_INIT_TIMEOUT_S seconds (default 120; 0 = wait without limit): HCCL_E_TIMEOUT, and the caller can
    // report the failure instead of hanging.  The helper thread stays behind in that case (it cannot be cancelled
    // inside the library call); it keeps its own copy of everything it touches.
    double limit_s = 120.0;
    if (const char *e = getenv("B200_HCCL_INIT_TIMEOUT_S")) limit_s = atof(e);
    int dev = -1;
    cudaGetDevice(&dev);   // the helper thread must bind the communicator to the caller's device
    struct Job {
        std::mutex mu;
        std::condition_variable cv;
        bool done = false;
        ncclComm_t comm = nullptr;
        ncclResult_t result = ncclInternalError;
    };
    auto job = std::make_shared<Job>();
    const auto init = nccl().CommInitRank;
    std::thread worker([job, init, id, nRanks, rank, dev] {
        if (dev >= 0) cudaSetDevice(dev);
        ncclComm_t c = nullptr;
        const ncclResult_t r = init(&c, (int)nRanks, id, (int)rank);
        std::lock_guard<std::mutex> lk(job->mu);
        job->comm = c; job->result = r; job->done = true;
        job->cv.notify_all();
    });
    {
        std::unique_lock<std::mutex> lk(job->mu);
        if (limit_s <= 0) job->cv.wait(lk, [&] { return job->done; });
        else if (!job->cv.wait_for(lk, std::chrono::duration<double>(limit_s), [&] { return job->done; })) {
            lk.unlock();
            worker.detach();
            fprintf(stderr, "[b200-hccl] HcclCommInitRootInfo: rank %u of %u gave up after %.1f s waiting for the other ranks\n",
                    rank, nRanks, limit_s);
            return HCCL_E_TIMEOUT;
        }
    }
    worker.join();
    if (job->result != ncclSuccess) return from_nccl(job->result);
    *comm = (HcclComm)job->comm;
    return HCCL_SUCCESS;
}

HcclResult HcclCommDestroy(HcclComm comm) {
    NEED_NCCL();
    if (!comm) return HCCL_E_PTR;
    p2p_forget(comm);
    return from_nccl(nccl().CommDestroy((ncclComm_t)comm));
}

HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                         HcclComm comm, aclrtStreamH stream) {
    NEED_NCCL();
    ncclDataType_t dt; ncclRedOp_t ro;
    if (!sendBuf || !recvBuf || !comm) return HCCL_E_PTR;
    if (!to_nccl(dataType, &dt) || !to_nccl(op, &ro)) return HCCL_E_NOT_SUPPORT;
    return from_nccl(nccl().AllReduce(sendBuf, recvBuf, count, dt, ro, (ncclComm_t)comm, (cudaStream_t)stream));
}

HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm,
                         aclrtStreamH stream) {
    NEED_NCCL();
    ncclDataType_t dt;
    if (!sendBuf || !recvBuf || !comm) return HCCL_E_PTR;
    if (!to_nccl(dataType, &dt)) return HCCL_E_NOT_SUPPORT;
    return from_nccl(nccl().AllGather(sendBuf, recvBuf, sendCount, dt, (ncclComm_t)comm, (cudaStream_t)stream));
}

HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op,
                             HcclComm comm, aclrtStreamH stream) {
    NEED_NCCL();
    ncclDataType_t dt; ncclRedOp_t ro;
    if (!sendBuf || !recvBuf || !comm) return HCCL_E_PTR;
    if (!to_nccl(dataType, &dt) || !to_nccl(op, &ro)) return HCCL_E_NOT_SUPPORT;
    return from_nccl(nccl().ReduceScatter(sendBuf, recvBuf, recvCount, dt, ro, (ncclComm_t)comm, (cudaStream_t)stream));
}

HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm,
                         aclrtStreamH stream) {
    NEED_NCCL();
    ncclDataType_t dt;
    if (!buf || !comm) return HCCL_E_PTR;
    if (!to_nccl(dataType, &dt)) return HCCL_E_NOT_SUPPORT;
    return from_nccl(nccl().Broadcast(buf, buf, count, dt, (int)root, (ncclComm_t)comm, (cudaStream_t)stream));
}

uint32_t HcclB200P2pStatus(void) { return p2p_status(); }
uint32_t HcclB200TestReceiverTimeout(uint64_t waitNs) { return p2p_test_poll_runs_out(waitNs); }
// for the gathering matmul of hccl_matmul.cpp
int hccl_gather_target(HcclComm comm, aclrtStreamH stream, P2pGatherTarget *t) {
    if (!nccl().ok || !comm) return 0;
    return p2p_gather_target(p2p_table(), comm, (cudaStream_t)stream, t) ? 1 : 0;
}
int hccl_gather_unpack(HcclComm comm, void *gathered, uint64_t elems_per_rank, aclrtStreamH stream) {
    return p2p_unpack(p2p_table(), comm, gathered, elems_per_rank, (cudaStream_t)stream);
}
int hccl_gather_reduce(HcclComm comm, void *out, uint64_t elems, int bf16, aclrtStreamH stream) {
    return p2p_reduce(p2p_table(), comm, out, elems, bf16 != 0, (cudaStream_t)stream);
}

HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize) {
    NEED_NCCL();
    if (!comm || !rankSize) return HCCL_E_PTR;
    int n = 0;
    ncclResult_t r = nccl().CommCount((ncclComm_t)comm, &n);
    *rankSize = (uint32_t)n;
    return from_nccl(r);
}

HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank) {
    NEED_NCCL();
    if (!comm || !rank) return HCCL_E_PTR;
    int n = 0;
    ncclResult_t r = nccl().CommUserRank((ncclComm_t)comm, &n);
    *rank = (uint32_t)n;
    return from_nccl(r);
}

}  // extern "C"
