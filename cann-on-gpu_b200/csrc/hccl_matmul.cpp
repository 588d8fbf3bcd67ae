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

// What phase 2 needs: the local operator's executor and what to all-reduce afterwards.  It rides in a
// wrapper plan of libascendcl.so, which owns it: destroying the plan (a caller that gives up after
// phase 1) ends up in free_allreduce.
struct AllReduceExecutor {
    aclOpExecutor *inner = nullptr;
    HcclComm comm = nullptr;
    const aclTensor *out = nullptr;
    bool weight_only = false;
};
void free_allreduce(void *p) {
    auto *w = static_cast<AllReduceExecutor *>(p);
    if (w->inner) aclDestroyAclOpExecutor(w->inner);
    delete w;
}

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
    *ex = aclnnB200CreateWrapperExecutor(w, free_allreduce);
    if (!*ex) { free_allreduce(w); return ACLNN_ERR_RUNTIME_ERROR; }
    return ACLNN_SUCCESS;
}

aclnnStatus run(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    auto *w = static_cast<AllReduceExecutor *>(aclnnB200WrapperPayload(e, 1));
    aclDestroyAclOpExecutor(e);   // phase 2 consumes the plan, whatever it was
    if (!w) return ACLNN_ERR_PARAM_INVALID;
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

// ---- W8A8 matmul -> all-reduce -> residual add + RMS norm (cuda/src/ops/matmul.cu:1222-1233,1344-1370).
// The matmul's partial output lives at the start of the caller's workspace (the reference allocates it
// with cudaMallocAsync inside phase 2); the norm is not linear, so the sum over ranks happens on that
// partial before it.
struct NormExecutor {
    const aclTensor *x = nullptr, *weight = nullptr, *scale = nullptr, *residual = nullptr, *gamma = nullptr;
    aclTensor *y = nullptr, *residual_sum = nullptr;
    double eps = 0.0;
    HcclComm comm = nullptr;
    uint64_t tmp_bytes = 0;
};
void free_norm(void *p) { delete static_cast<NormExecutor *>(p); }

// A tensor of y's shape and type over `data`.
aclTensor *like(const aclTensor *y, void *data, uint64_t *count, aclDataType *dt) {
    int64_t *dims = nullptr;
    uint64_t nd = 0;
    if (aclGetViewShape(y, &dims, &nd) != ACLNN_SUCCESS || aclGetDataType(y, dt) != ACLNN_SUCCESS) return nullptr;
    *count = 1;
    for (uint64_t i = 0; i < nd; ++i) *count *= (uint64_t)dims[i];
    return aclCreateTensor(dims, nd, *dt, nullptr, 0, ACL_FORMAT_ND, dims, nd, data);
}

aclnnStatus norm_plan(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, const aclTensor *residual,
                      const aclTensor *gamma, double eps, HcclComm comm, aclTensor *y, aclTensor *residual_sum, uint64_t *ws,
                      aclOpExecutor **ex) {
    if (!x || !weight || !scale || !residual || !y || !residual_sum || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    void *ydata = nullptr;
    if (aclGetRawTensorAddr(y, &ydata) != ACLNN_SUCCESS || !ydata) return ACLNN_ERR_PARAM_NULLPTR;
    uint64_t count = 0;
    aclDataType dt = ACL_DT_UNDEFINED;
    aclTensor *probe = like(y, ydata, &count, &dt);   // same shape and type as the partial output
    if (!probe) return ACLNN_ERR_PARAM_INVALID;
    HcclDataType ht;
    aclnnStatus st = hccl_type(dt, &ht) ? ACLNN_SUCCESS : ACLNN_ERR_PARAM_INVALID;
    uint64_t inner_ws = 0, norm_ws = 0;
    aclOpExecutor *inner = nullptr;
    if (st == ACLNN_SUCCESS) st = aclnnQuantMatmulGetWorkspaceSize(x, weight, scale, probe, &inner_ws, &inner);
    if (st == ACLNN_SUCCESS) {
        aclDestroyAclOpExecutor(inner);
        st = aclnnAddRmsNormGetWorkspaceSize(probe, residual, gamma, eps, y, residual_sum, &norm_ws, &inner);
        if (st == ACLNN_SUCCESS) aclDestroyAclOpExecutor(inner);
    }
    aclDestroyTensor(probe);
    if (st != ACLNN_SUCCESS) return st;
    auto *n = new NormExecutor();
    n->x = x; n->weight = weight; n->scale = scale; n->residual = residual; n->gamma = gamma; n->y = y; n->residual_sum = residual_sum;
    n->eps = eps; n->comm = comm;
    n->tmp_bytes = (count * (dt == ACL_FLOAT ? 4 : 2) + 255) / 256 * 256;
    *ws = n->tmp_bytes + inner_ws;
    *ex = aclnnB200CreateWrapperExecutor(n, free_norm);
    if (!*ex) { delete n; return ACLNN_ERR_RUNTIME_ERROR; }
    return ACLNN_SUCCESS;
}

aclnnStatus norm_run(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    auto *np = static_cast<NormExecutor *>(aclnnB200WrapperPayload(e, 1));
    aclDestroyAclOpExecutor(e);
    if (!np) return ACLNN_ERR_PARAM_INVALID;
    const NormExecutor n = *np;
    delete np;
    if (!ws || wsz < n.tmp_bytes) return ACLNN_ERR_PARAM_INVALID;
    uint64_t count = 0;
    aclDataType dt = ACL_DT_UNDEFINED;
    aclTensor *tmp = like(n.y, ws, &count, &dt);
    if (!tmp) return ACLNN_ERR_PARAM_INVALID;
    uint64_t need = 0;
    aclOpExecutor *inner = nullptr;
    aclnnStatus st = aclnnQuantMatmulGetWorkspaceSize(n.x, n.weight, n.scale, tmp, &need, &inner);
    if (st == ACLNN_SUCCESS) {
        if (need > wsz - n.tmp_bytes) { aclDestroyAclOpExecutor(inner); st = ACLNN_ERR_PARAM_INVALID; }
        else st = aclnnQuantMatmul(static_cast<char *>(ws) + n.tmp_bytes, wsz - n.tmp_bytes, inner, s);
    }
    HcclDataType ht;
    if (st == ACLNN_SUCCESS && n.comm && count > 0) {
        if (!hccl_type(dt, &ht) || HcclAllReduce(ws, ws, count, ht, HCCL_REDUCE_SUM, n.comm, s) != HCCL_SUCCESS) st = ACLNN_ERR_RUNTIME_ERROR;
    }
    if (st == ACLNN_SUCCESS) {
        st = aclnnAddRmsNormGetWorkspaceSize(tmp, n.residual, n.gamma, n.eps, n.y, n.residual_sum, &need, &inner);
        if (st == ACLNN_SUCCESS) st = aclnnAddRmsNorm(nullptr, 0, inner, s);
    }
    aclDestroyTensor(tmp);
    return st;
}

}  // namespace

extern "C" {

aclnnStatus aclnnQuantMatmulAllReduceAddRmsNormGetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *scale,
        const aclTensor *residual, const aclTensor *gamma, double eps, HcclComm comm, aclTensor *y, aclTensor *residualSum,
        uint64_t *ws, aclOpExecutor **ex) {
    return norm_plan(x, weight, scale, residual, gamma, eps, comm, y, residualSum, ws, ex);
}
aclnnStatus aclnnQuantMatmulAllReduceAddRmsNorm(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return norm_run(ws, wsz, e, s); }

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
