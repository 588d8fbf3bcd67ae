// Shared host-side definitions of the quantized-matmul library: the concrete aclTensor /
// aclOpExecutor objects behind the opaque handles, error mapping and small dtype helpers.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "acl/acl.h"
#include "aclnn/acl_meta.h"
#include "aclnnop/aclnn_quant_matmul.h"

// Host metadata over a caller-owned device buffer (same role as the reference's aclTensor,
// cuda/src/internal.h:30-50).
struct aclTensor {
    std::vector<int64_t> viewDims, strides, storageDims;
    int64_t offset = 0;  // element offset into `data`
    aclDataType dtype = ACL_DT_UNDEFINED;
    aclFormat format = ACL_FORMAT_ND;
    void *data = nullptr;

    int64_t numel() const {
        int64_t n = 1;
        for (auto d : viewDims) n *= d;
        return n;
    }
    bool contiguous() const {
        int64_t s = 1;
        for (int i = (int)viewDims.size() - 1; i >= 0; --i) {
            if (viewDims[i] != 1 && strides[i] != s) return false;
            s *= viewDims[i];
        }
        return true;
    }
    int rank() const { return (int)viewDims.size(); }
};

struct aclScalar {
    double v = 0.0;
    aclDataType dtype = ACL_DT_UNDEFINED;
};
struct aclIntArray {
    std::vector<int64_t> v;
};
struct aclTensorList {
    std::vector<const aclTensor *> v;
};

// CUDA error -> aclError: 0, or 500000 + the CUDA code (cuda/src/internal.h:22-27 of the reference).
inline aclError acl_from_cuda(cudaError_t e) { return e == cudaSuccess ? ACL_SUCCESS : (aclError)(500000 + (int)e); }
#define ACL_CUDA(call)                                                                                         \
    do {                                                                                                       \
        cudaError_t _e = (call);                                                                               \
        if (_e != cudaSuccess) {                                                                               \
            fprintf(stderr, "[b200-qmm] %s:%d CUDA error %d (%s)\n", __FILE__, __LINE__, (int)_e,              \
                    cudaGetErrorString(_e));                                                                   \
            return acl_from_cuda(_e);                                                                          \
        }                                                                                                      \
    } while (0)

// Bytes of one element; sub-byte types return the sentinel 1 so that tensors of them can be created
// (cuda/src/internal.h:147-162 of the reference).  Packed sizes are computed where they are used.
inline size_t dtype_size(aclDataType t) {
    switch (t) {
        case ACL_FLOAT: case ACL_INT32: case ACL_UINT32: return 4;
        case ACL_FLOAT16: case ACL_BF16: case ACL_INT16: case ACL_UINT16: return 2;
        case ACL_INT8: case ACL_UINT8: case ACL_BOOL: return 1;
        case ACL_FLOAT8_E4M3FN: case ACL_FLOAT8_E5M2: case ACL_FLOAT8_E8M0: case ACL_HIFLOAT8: return 1;
        case ACL_INT64: case ACL_UINT64: case ACL_DOUBLE: return 8;
        case ACL_FLOAT4_E2M1: case ACL_FLOAT4_E1M2: case ACL_FLOAT6_E2M3: case ACL_FLOAT6_E3M2: return 1;
        case ACL_INT4: return 1;
        default: return 0;
    }
}

inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }
