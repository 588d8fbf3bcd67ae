// aclrt* runtime subset over the CUDA runtime: what a standalone client of the quantized-matmul
// operators needs (device, stream, event, memory).  Mirrors the call contract of the reference's
// cuda/src/runtime.cu:45-134.
#include <new>
#include <map>
#include <mutex>
#include <unordered_map>

#include "internal.h"

namespace {

// Device-memory pool: freed blocks are kept and handed back to the next request they can hold
// (cudaMalloc/cudaFree synchronise the device, which clients that allocate a workspace per call
// cannot afford).  Requests are rounded to 512 B below 1 MiB and to 2 MiB above; a cached block is
// reused when it is at most 2x the request.  B200_ACL_NO_POOL=1 turns the pool off.
class DevicePool {
public:
    cudaError_t get(void **p, size_t n) {
        size_t want = round_size(n);
        int dev = 0;
        cudaGetDevice(&dev);
        if (enabled_) {
            std::lock_guard<std::mutex> g(mu_);
            auto &fl = free_[dev];
            auto it = fl.lower_bound(want);
            if (it != fl.end() && it->first <= 2 * want) {
                *p = it->second;
                live_[*p] = {it->first, dev};
                fl.erase(it);
                return cudaSuccess;
            }
        }
        cudaError_t e = cudaMalloc(p, want);
        if (e != cudaSuccess && enabled_) {  // give cached blocks back to the driver and retry once
            trim(dev);
            e = cudaMalloc(p, want);
        }
        if (e == cudaSuccess && enabled_) {
            std::lock_guard<std::mutex> g(mu_);
            live_[*p] = {want, dev};
        }
        return e;
    }
    cudaError_t put(void *p) {
        if (!p) return cudaSuccess;
        if (enabled_) {
            std::lock_guard<std::mutex> g(mu_);
            auto it = live_.find(p);
            if (it != live_.end()) {
                free_[it->second.dev].emplace(it->second.bytes, p);
                live_.erase(it);
                return cudaSuccess;
            }
        }
        return cudaFree(p);
    }

private:
    struct Block { size_t bytes; int dev; };
    static size_t round_size(size_t n) {
        if (n == 0) n = 1;
        const size_t small = 512, big = (size_t)2 << 20;
        return n < ((size_t)1 << 20) ? (n + small - 1) / small * small : (n + big - 1) / big * big;
    }
    void trim(int dev) {
        std::lock_guard<std::mutex> g(mu_);
        for (auto &kv : free_[dev]) cudaFree(kv.second);
        free_[dev].clear();
    }
    std::mutex mu_;
    std::unordered_map<int, std::multimap<size_t, void *>> free_;
    std::unordered_map<void *, Block> live_;
    bool enabled_ = getenv("B200_ACL_NO_POOL") == nullptr;
};

DevicePool &pool() {
    static DevicePool *p = new DevicePool();  // never destroyed: the context outlives static dtors
    return *p;
}

cudaMemcpyKind copy_kind(aclrtMemcpyKind k) {
    switch (k) {
        case ACL_MEMCPY_HOST_TO_HOST: return cudaMemcpyHostToHost;
        case ACL_MEMCPY_HOST_TO_DEVICE: return cudaMemcpyHostToDevice;
        case ACL_MEMCPY_DEVICE_TO_HOST: return cudaMemcpyDeviceToHost;
        case ACL_MEMCPY_DEVICE_TO_DEVICE: return cudaMemcpyDeviceToDevice;
    }
    return cudaMemcpyDefault;
}

}  // namespace

extern "C" {

aclError aclInit(const char *) { return acl_from_cuda(cudaFree(0)); }
aclError aclFinalize(void) { return ACL_SUCCESS; }
aclError aclrtSetDevice(int32_t deviceId) { return acl_from_cuda(cudaSetDevice(deviceId)); }
aclError aclrtResetDevice(int32_t) { return ACL_SUCCESS; }
aclError aclrtGetDevice(int32_t *deviceId) { return deviceId ? acl_from_cuda(cudaGetDevice(deviceId)) : ACLNN_ERR_PARAM_NULLPTR; }
aclError aclrtGetDeviceCount(uint32_t *count) {
    if (!count) return ACLNN_ERR_PARAM_NULLPTR;
    int n = 0;
    ACL_CUDA(cudaGetDeviceCount(&n));
    *count = (uint32_t)n;
    return ACL_SUCCESS;
}
aclError aclrtGetRunMode(aclrtRunMode *runMode) {
    if (!runMode) return ACLNN_ERR_PARAM_NULLPTR;
    *runMode = ACL_HOST;
    return ACL_SUCCESS;
}

aclError aclrtCreateStream(aclrtStream *stream) {
    if (!stream) return ACLNN_ERR_PARAM_NULLPTR;
    return acl_from_cuda(cudaStreamCreateWithFlags(reinterpret_cast<cudaStream_t *>(stream), cudaStreamNonBlocking));
}
aclError aclrtDestroyStream(aclrtStream stream) { return acl_from_cuda(cudaStreamDestroy((cudaStream_t)stream)); }
aclError aclrtSynchronizeStream(aclrtStream stream) { return acl_from_cuda(cudaStreamSynchronize((cudaStream_t)stream)); }
aclError aclrtSynchronizeDevice(void) { return acl_from_cuda(cudaDeviceSynchronize()); }

aclError aclrtCreateEvent(aclrtEvent *event) {
    if (!event) return ACLNN_ERR_PARAM_NULLPTR;
    return acl_from_cuda(cudaEventCreate(reinterpret_cast<cudaEvent_t *>(event)));
}
aclError aclrtDestroyEvent(aclrtEvent event) { return acl_from_cuda(cudaEventDestroy((cudaEvent_t)event)); }
aclError aclrtRecordEvent(aclrtEvent event, aclrtStream stream) {
    return acl_from_cuda(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
}
aclError aclrtStreamWaitEvent(aclrtStream stream, aclrtEvent event) {
    return acl_from_cuda(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
}
aclError aclrtSynchronizeEvent(aclrtEvent event) { return acl_from_cuda(cudaEventSynchronize((cudaEvent_t)event)); }
aclError aclrtEventElapsedTime(float *ms, aclrtEvent startEvent, aclrtEvent endEvent) {
    if (!ms) return ACLNN_ERR_PARAM_NULLPTR;
    return acl_from_cuda(cudaEventElapsedTime(ms, (cudaEvent_t)startEvent, (cudaEvent_t)endEvent));
}

// ---- stream capture and replay (reference: cuda/src/runtime.cu:138-189) ---------------------------
// A model is a captured CUDA graph with its executable instance.
namespace {
struct CapturedModel {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    ~CapturedModel() {
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
    }
};
}  // namespace

aclError aclmdlRICaptureBegin(aclrtStream stream, aclmdlRICaptureMode mode) {
    const cudaStreamCaptureMode m = mode == ACL_MODEL_RI_CAPTURE_MODE_THREAD_LOCAL ? cudaStreamCaptureModeThreadLocal
                                  : mode == ACL_MODEL_RI_CAPTURE_MODE_RELAXED    ? cudaStreamCaptureModeRelaxed
                                                                                 : cudaStreamCaptureModeGlobal;
    return acl_from_cuda(cudaStreamBeginCapture((cudaStream_t)stream, m));
}
aclError aclmdlRICaptureGetInfo(aclrtStream stream, aclmdlRICaptureStatus *status, aclmdlRI *modelRI) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    const cudaError_t e = cudaStreamIsCapturing((cudaStream_t)stream, &cs);
    if (status) {
        *status = cs == cudaStreamCaptureStatusActive        ? ACL_MODEL_RI_CAPTURE_STATUS_ACTIVE
                : cs == cudaStreamCaptureStatusInvalidated   ? ACL_MODEL_RI_CAPTURE_STATUS_INVALIDATED
                                                             : ACL_MODEL_RI_CAPTURE_STATUS_NONE;
    }
    if (modelRI) *modelRI = nullptr;   // a model exists only after aclmdlRICaptureEnd
    return acl_from_cuda(e);
}
aclError aclmdlRICaptureEnd(aclrtStream stream, aclmdlRI *modelRI) {
    if (!modelRI) return ACLNN_ERR_PARAM_NULLPTR;
    *modelRI = nullptr;
    CapturedModel *m = new (std::nothrow) CapturedModel();
    if (!m) return ACLNN_ERR_RUNTIME_ERROR;
    cudaError_t e = cudaStreamEndCapture((cudaStream_t)stream, &m->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&m->exec, m->graph, 0);
    if (e != cudaSuccess) { delete m; return acl_from_cuda(e); }
    *modelRI = m;
    return ACL_SUCCESS;
}
aclError aclmdlRIExecuteAsync(aclmdlRI modelRI, aclrtStream stream) {
    if (!modelRI) return ACLNN_ERR_PARAM_NULLPTR;
    return acl_from_cuda(cudaGraphLaunch(static_cast<CapturedModel *>(modelRI)->exec, (cudaStream_t)stream));
}
aclError aclmdlRIExecute(aclmdlRI modelRI, int32_t /*timeout*/) {
    if (!modelRI) return ACLNN_ERR_PARAM_NULLPTR;
    const cudaError_t e = cudaGraphLaunch(static_cast<CapturedModel *>(modelRI)->exec, nullptr);
    return acl_from_cuda(e == cudaSuccess ? cudaStreamSynchronize(nullptr) : e);
}
aclError aclmdlRIDestroy(aclmdlRI modelRI) {
    delete static_cast<CapturedModel *>(modelRI);
    return ACL_SUCCESS;
}

aclError aclrtMalloc(void **devPtr, size_t size, aclrtMemMallocPolicy) {
    if (!devPtr) return ACLNN_ERR_PARAM_NULLPTR;
    return acl_from_cuda(pool().get(devPtr, size));
}
aclError aclrtFree(void *devPtr) { return acl_from_cuda(pool().put(devPtr)); }
aclError aclrtMallocHost(void **hostPtr, size_t size) {
    if (!hostPtr) return ACLNN_ERR_PARAM_NULLPTR;
    return acl_from_cuda(cudaMallocHost(hostPtr, size));
}
aclError aclrtFreeHost(void *hostPtr) { return acl_from_cuda(cudaFreeHost(hostPtr)); }

aclError aclrtMemcpy(void *dst, size_t destMax, const void *src, size_t count, aclrtMemcpyKind kind) {
    if (count > destMax) return ACLNN_ERR_PARAM_INVALID;
    return acl_from_cuda(cudaMemcpy(dst, src, count, copy_kind(kind)));
}
aclError aclrtMemcpyAsync(void *dst, size_t destMax, const void *src, size_t count, aclrtMemcpyKind kind,
                          aclrtStream stream) {
    if (count > destMax) return ACLNN_ERR_PARAM_INVALID;
    return acl_from_cuda(cudaMemcpyAsync(dst, src, count, copy_kind(kind), (cudaStream_t)stream));
}
aclError aclrtMemset(void *devPtr, size_t maxCount, int32_t value, size_t count) {
    if (count > maxCount) return ACLNN_ERR_PARAM_INVALID;
    return acl_from_cuda(cudaMemset(devPtr, value, count));
}
size_t aclDataTypeSize(aclDataType dataType) { return dtype_size(dataType); }

}  // extern "C"
