/*
 * acl/acl.h -- minimal, self-declared subset of the AscendCL runtime header.
 *
 * The reference project compiles against the vendor's acl/acl.h, which it does not ship
 * (include/README.md:14-17 of the reference).  Only the symbols the quantized-matmul path and its
 * test clients use are declared here (runtime.cu:45-134 of the reference maps each one to the CUDA
 * runtime).  Enumerator values are self-consistent inside this library; when this library is
 * built against the vendor header instead, that header wins (same names, same argument order).
 */
#ifndef B200_ACL_ACL_H
#define B200_ACL_ACL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef ACL_FUNC_VISIBILITY
#define ACL_FUNC_VISIBILITY __attribute__((visibility("default")))
#endif

typedef int aclError;
#define ACL_SUCCESS 0
#define ACL_ERROR_NONE 0

typedef void *aclrtStream;
typedef void *aclrtEvent;
typedef void *aclrtContext;

typedef enum {
    ACL_DT_UNDEFINED = -1,
    ACL_FLOAT = 0,
    ACL_FLOAT16 = 1,
    ACL_INT8 = 2,
    ACL_INT32 = 3,
    ACL_UINT8 = 4,
    ACL_INT16 = 6,
    ACL_UINT16 = 7,
    ACL_UINT32 = 8,
    ACL_INT64 = 9,
    ACL_UINT64 = 10,
    ACL_DOUBLE = 11,
    ACL_BOOL = 12,
    ACL_BF16 = 27,
    ACL_INT4 = 29,
    ACL_HIFLOAT8 = 34,
    ACL_FLOAT8_E5M2 = 35,
    ACL_FLOAT8_E4M3FN = 36,
    ACL_FLOAT8_E8M0 = 37,
    ACL_FLOAT6_E3M2 = 38,
    ACL_FLOAT6_E2M3 = 39,
    ACL_FLOAT4_E2M1 = 40,
    ACL_FLOAT4_E1M2 = 41
} aclDataType;

typedef enum {
    ACL_FORMAT_UNDEFINED = -1,
    ACL_FORMAT_NCHW = 0,
    ACL_FORMAT_NHWC = 1,
    ACL_FORMAT_ND = 2,
    ACL_FORMAT_FRACTAL_NZ = 29
} aclFormat;

typedef enum {
    ACL_MEM_MALLOC_HUGE_FIRST = 0,
    ACL_MEM_MALLOC_HUGE_ONLY = 1,
    ACL_MEM_MALLOC_NORMAL_ONLY = 2
} aclrtMemMallocPolicy;

typedef enum {
    ACL_MEMCPY_HOST_TO_HOST = 0,
    ACL_MEMCPY_HOST_TO_DEVICE = 1,
    ACL_MEMCPY_DEVICE_TO_HOST = 2,
    ACL_MEMCPY_DEVICE_TO_DEVICE = 3
} aclrtMemcpyKind;

typedef enum { ACL_DEVICE = 0, ACL_HOST = 1 } aclrtRunMode;

/* Process / device / stream lifetime (reference: cuda/src/runtime.cu:47-88). */
ACL_FUNC_VISIBILITY aclError aclInit(const char *configPath);
ACL_FUNC_VISIBILITY aclError aclFinalize(void);
ACL_FUNC_VISIBILITY aclError aclrtSetDevice(int32_t deviceId);
ACL_FUNC_VISIBILITY aclError aclrtResetDevice(int32_t deviceId);
ACL_FUNC_VISIBILITY aclError aclrtGetDevice(int32_t *deviceId);
ACL_FUNC_VISIBILITY aclError aclrtGetDeviceCount(uint32_t *count);
ACL_FUNC_VISIBILITY aclError aclrtGetRunMode(aclrtRunMode *runMode);
ACL_FUNC_VISIBILITY aclError aclrtCreateStream(aclrtStream *stream);
ACL_FUNC_VISIBILITY aclError aclrtDestroyStream(aclrtStream stream);
ACL_FUNC_VISIBILITY aclError aclrtSynchronizeStream(aclrtStream stream);
ACL_FUNC_VISIBILITY aclError aclrtSynchronizeDevice(void);

/* Events (reference: cuda/src/runtime.cu:90-101). */
ACL_FUNC_VISIBILITY aclError aclrtCreateEvent(aclrtEvent *event);
ACL_FUNC_VISIBILITY aclError aclrtDestroyEvent(aclrtEvent event);
ACL_FUNC_VISIBILITY aclError aclrtRecordEvent(aclrtEvent event, aclrtStream stream);
/* reference: cuda/src/runtime.cu:221. */
ACL_FUNC_VISIBILITY aclError aclrtStreamWaitEvent(aclrtStream stream, aclrtEvent event);
ACL_FUNC_VISIBILITY aclError aclrtSynchronizeEvent(aclrtEvent event);
ACL_FUNC_VISIBILITY aclError aclrtEventElapsedTime(float *ms, aclrtEvent startEvent, aclrtEvent endEvent);

/* Stream capture and replay (reference: cuda/src/runtime.cu:138-189; used as in tests/test_graph.cpp:
 * warm up, capture a sequence of two-phase operator calls that reuse a caller-owned workspace, then
 * replay the model).  Phase 1 runs on the host at capture time only; phase 2 of every operator of
 * this library enqueues without allocating or synchronising, so it can be captured. */
typedef void *aclmdlRI;
typedef enum {
    ACL_MODEL_RI_CAPTURE_MODE_GLOBAL = 0,
    ACL_MODEL_RI_CAPTURE_MODE_THREAD_LOCAL = 1,
    ACL_MODEL_RI_CAPTURE_MODE_RELAXED = 2
} aclmdlRICaptureMode;
typedef enum {
    ACL_MODEL_RI_CAPTURE_STATUS_NONE = 0,
    ACL_MODEL_RI_CAPTURE_STATUS_ACTIVE = 1,
    ACL_MODEL_RI_CAPTURE_STATUS_INVALIDATED = 2
} aclmdlRICaptureStatus;
ACL_FUNC_VISIBILITY aclError aclmdlRICaptureBegin(aclrtStream stream, aclmdlRICaptureMode mode);
ACL_FUNC_VISIBILITY aclError aclmdlRICaptureGetInfo(aclrtStream stream, aclmdlRICaptureStatus *status, aclmdlRI *modelRI);
ACL_FUNC_VISIBILITY aclError aclmdlRICaptureEnd(aclrtStream stream, aclmdlRI *modelRI);
ACL_FUNC_VISIBILITY aclError aclmdlRIExecuteAsync(aclmdlRI modelRI, aclrtStream stream);
ACL_FUNC_VISIBILITY aclError aclmdlRIExecute(aclmdlRI modelRI, int32_t timeout);
ACL_FUNC_VISIBILITY aclError aclmdlRIDestroy(aclmdlRI modelRI);

/* Device / pinned-host memory (reference: cuda/src/runtime.cu:103-134). */
ACL_FUNC_VISIBILITY aclError aclrtMalloc(void **devPtr, size_t size, aclrtMemMallocPolicy policy);
ACL_FUNC_VISIBILITY aclError aclrtFree(void *devPtr);
ACL_FUNC_VISIBILITY aclError aclrtMallocHost(void **hostPtr, size_t size);
ACL_FUNC_VISIBILITY aclError aclrtFreeHost(void *hostPtr);
ACL_FUNC_VISIBILITY aclError aclrtMemcpy(void *dst, size_t destMax, const void *src, size_t count,
                                         aclrtMemcpyKind kind);
ACL_FUNC_VISIBILITY aclError aclrtMemcpyAsync(void *dst, size_t destMax, const void *src, size_t count,
                                              aclrtMemcpyKind kind, aclrtStream stream);
ACL_FUNC_VISIBILITY aclError aclrtMemset(void *devPtr, size_t maxCount, int32_t value, size_t count);
ACL_FUNC_VISIBILITY size_t aclDataTypeSize(aclDataType dataType);

#ifdef __cplusplus
}
#endif
#endif
