// Quantized matmuls followed by an all-reduce over a communicator (K-split tensor parallelism): the
// local operator of libascendcl.so, then HcclAllReduce(SUM) of the output on the caller's stream.
// Scales are linear over the K reduction, so summing the ranks' scaled partial outputs equals
// scaling the full sum.  comm == NULL gives the local result (exact for one rank).
//
// Same contract as the reference's cuda/src/ops/mc2_ext.cu:67-87,185-195 and
// cuda/src/ops/matmul.cu:1304-1319, but the state travels in the executor handed back to the
// caller instead of a process-wide map (the reference's maps are not thread-safe).
#include <cstdint>

#include "aclnnop/aclnn_quant_matmul_mc2.h"

namespace {

constexpr uint64_t WRAP_MAGIC = 0x4232303048434c41ull;

// What phase 2 needs: the local operator's executor and what to all-reduce afterwards.
struct AllReduceExecutor {
    uint64_t magic = WRAP_MAGIC;
    aclOpExecutor *inner = nullptr;
    HcclComm comm = nullptr;
    const aclTensor *out = nullptr;
    bool weight_only = false;
};

bool hccl_type(aclDataType d, HcclDataType *t) {
    switch (d) {
        case ACL_FLOAT: *t = HCCL_DATA_TYPE_FP32; return true;
        case ACL_FLOAT16: *t = HCCL_DATA_TYPE_FP16; return true;
        case ACL_BF16: *t = HCCL_DATA_TYPE_BFP16; return true;
        default: return false;
    }
}

aclnnStatus wrap(aclnnStatus st, aclOpExecutor *inner, HcclComm comm, const aclTensor *out, bool weight_only, aclOpExecutor **ex) {
    if (st != ACLNN_SUCCESS) return st;
    aclDataType dt;
    HcclDataType ht;
    if (aclGetDataType(out, &dt) != ACLNN_SUCCESS || (comm && !hccl_type(dt, &ht))) {
        aclDestroyAclOpExecutor(inner);
        return ACLNN_ERR_PARAM_INVALID;
    }
    auto *w = new AllReduceExecutor();
    w->inner = inner; w->comm = comm; w->out = out; w->weight_only = weight_only;
    *ex = reinterpret_cast<aclOpExecutor *>(w);
    return ACLNN_SUCCESS;
}

aclnnStatus run(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) {
    auto *w = reinterpret_cast<AllReduceExecutor *>(e);
    if (!w || w->magic != WRAP_MAGIC) return ACLNN_ERR_PARAM_INVALID;
    // read what the all-reduce needs before the local operator runs: the tensors may go away after phase 2
    void *data = nullptr;
    int64_t *dims = nullptr;
    uint64_t nd = 0;
    aclDataType dt = ACL_DT_UNDEFINED;
    aclnnStatus st = aclGetRawTensorAddr(w->out, &data);
    if (st == ACLNN_SUCCESS) st = aclGetViewShape(w->out, &dims, &nd);
    if (st == ACLNN_SUCCESS) st = aclGetDataType(w->out, &dt);
    uint64_t count = 1;
    for (uint64_t i = 0; st == ACLNN_SUCCESS && i < nd; ++i) count *= (uint64_t)dims[i];
    aclOpExecutor *inner = w->inner;
    HcclComm comm = w->comm;
    const bool weight_only = w->weight_only;
    w->magic = 0;
    delete w;
    if (st != ACLNN_SUCCESS) {
        aclDestroyAclOpExecutor(inner);
        return st;
    }
    st = weight_only ? aclnnWeightQuantBatchMatmul(ws, wsz, inner, s) : aclnnQuantMatmul(ws, wsz, inner, s);
    if (st == ACLNN_SUCCESS && comm && count > 0) {
        HcclDataType ht;
        if (!hccl_type(dt, &ht)) return ACLNN_ERR_PARAM_INVALID;
        if (HcclAllReduce(data, data, count, ht, HCCL_REDUCE_SUM, comm, s) != HCCL_SUCCESS) st = ACLNN_ERR_RUNTIME_ERROR;
    }
    return st;
}

}  // namespace

extern "C" {

#define QMM_ALLREDUCE(NAME)                                                                                          \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, HcclComm comm, \
                                       aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {                           \
        if (!x || !weight || !scale || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;                           \
        aclOpExecutor *inner = nullptr;                                                                              \
        const aclnnStatus st = aclnnQuantMatmulGetWorkspaceSize(x, weight, scale, out, ws, &inner);                  \
        return wrap(st, inner, comm, out, false, ex);                                                                \
    }                                                                                                                \
    aclnnStatus NAME(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return run(ws, wsz, e, s); }
QMM_ALLREDUCE(aclnnQuantMatmulAllReduce)
QMM_ALLREDUCE(aclnnQuantMatmulAllReduceV2)
QMM_ALLREDUCE(aclnnQuantMatmulAllReduceV3)
QMM_ALLREDUCE(aclnnQuantMatmulAllReduceV4)

aclnnStatus aclnnWeightQuantMatmulAllReduceGetWorkspaceSize(const aclTensor *x, const aclTensor *weight,
        const aclTensor *antiquantScale, const aclTensor *antiquantOffset, HcclComm comm, aclTensor *out, uint64_t *ws,
        aclOpExecutor **ex) {
    if (!x || !weight || !antiquantScale || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    aclOpExecutor *inner = nullptr;
    const aclnnStatus st = aclnnWeightQuantBatchMatmulGetWorkspaceSize(x, weight, antiquantScale, antiquantOffset, out, ws, &inner);
    return wrap(st, inner, comm, out, true, ex);
}
aclnnStatus aclnnWeightQuantMatmulAllReduce(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return run(ws, wsz, e, s); }

}  // extern "C"
