// One-shot execution plan built by every ...GetWorkspaceSize call and consumed by the matching
// execute call (same life cycle as the reference's aclOpExecutor, cuda/src/internal.h:60-85, but
// all state lives in the plan -- no global maps -- so concurrent callers do not interfere).
#pragma once

#include "internal.h"

enum PlanOp : int {
    PLAN_WQBMM = 1,   // weight-only quantized matmul (W8A16 / W4A16)
    PLAN_QMM,         // W8A8 quantized matmul
    PLAN_MX,          // MX block-scaled matmul
    PLAN_INT4_PACK,   // two int8 -> one packed byte
    PLAN_COPY,        // weight copy (identity pre-pack)
    PLAN_PACK_NZ,     // int4 weight [K,N] -> tile-packed layout
    PLAN_WIDEN_FP4,   // fp4 weight -> one e4m3 byte per element
    PLAN_WEIGHT_SIZE, // element count of a weight shape
    PLAN_CAST,        // element-wise dtype cast
    PLAN_QPARAM,      // fp32 scale (+ offset) -> packed int64 quant parameter
    PLAN_DYNQUANT,    // per-token dynamic int8 quantiser
    PLAN_SWIGLUQUANT, // SwiGLU fused with the per-token quantiser
    PLAN_MXQUANT,     // block-wise power-of-two-scale int8 quantiser
    PLAN_ADDRMSNORM,  // residual add + RMS norm (tail of the all-reduce matmuls)
    PLAN_WRAPPER,     // plan of a composite operator living in another library (payload + deleter below)
};

// Kernel families a plan can select.
enum PlanPath : int {
    PATH_GENERIC = 0,  // bounds-checked CUDA-core tile kernel: any shape, any dtype mix
    PATH_GEMV,         // HBM-bound streaming kernel for very small M (CUDA cores, split-K)
    PATH_TC,           // tcgen05 tensor-core kernel (TMA + TMEM), weights on the MMA M side
};

struct aclOpExecutor {
    PlanOp op = PLAN_WQBMM;
    PlanPath path = PATH_GENERIC;
    // Tensors stay owned by the caller; their data pointers are read when the plan executes, so a
    // caller may re-point a tensor (aclSetRawTensorAddr) between the two phases.
    const aclTensor *a = nullptr;        // x / self
    const aclTensor *b = nullptr;        // weight / other
    const aclTensor *scale = nullptr;    // antiquantScale / deq scale / selfScale
    const aclTensor *scale2 = nullptr;   // antiquantOffset / otherScale
    const aclTensor *bias = nullptr;
    const aclTensor *pertoken = nullptr;
    aclTensor *out = nullptr;
    aclTensor *out2 = nullptr;            // second output (per-token scales of the dynamic quantiser)
    int64_t batch = 1, m = 0, n = 0, k = 0;
    int64_t group = 0;          // rows of K per antiquant scale row (K for per-channel)
    bool b_transposed = false;  // weight stored [N,K]
    bool accumulate = false;    // out += result
    int split_k = 1;
    uint64_t ws_bytes = 0;
    aclDataType cast_to = ACL_DT_UNDEFINED;
    double eps = 0.0;            // PLAN_ADDRMSNORM
    std::vector<int64_t> shape;  // PLAN_WEIGHT_SIZE
    // PLAN_WRAPPER: state of a composite operator (the all-reduce matmuls of libhccl.so).  The executor
    // owns it: aclDestroyAclOpExecutor calls payload_free(payload), so a plan abandoned after phase 1
    // is released correctly, and the plain execute entries refuse such a plan.
    void *payload = nullptr;
    void (*payload_free)(void *) = nullptr;
    ~aclOpExecutor() { if (payload && payload_free) payload_free(payload); }
};
