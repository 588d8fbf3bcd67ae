// The aclnn two-phase operator surface of the quantized-matmul family: argument validation, plan
// construction (kernel path, split-K, workspace bytes) and execution on the caller's stream.
//
// Call contract follows the reference (cuda/src/ops/matmul.cu:758-859, cuda/src/ops/quant.cu:196-326):
// phase 1 is host-only and returns 161001 for null arguments and 161002 for unsupported types or
// shapes; phase 2 enqueues on the stream, never synchronises or allocates, reports launch errors as
// 361001 and consumes the executor.
#include <atomic>
#include <cstdint>
#include <cstring>
#include <new>

#include "aclnnop/aclnn_quant_matmul.h"
#include "executor.h"
#include "kernels.h"

using namespace qmm;

namespace {

int elem_type(aclDataType t) {
    switch (t) {
        case ACL_FLOAT: return ET_F32;
        case ACL_FLOAT16: return ET_F16;
        case ACL_BF16: return ET_BF16;
        case ACL_INT8: return ET_I8;
        case ACL_UINT8: return ET_U8;
        case ACL_INT4: return ET_I4;
        case ACL_INT32: return ET_I32;
        case ACL_FLOAT8_E4M3FN: return ET_E4M3;
        case ACL_FLOAT8_E5M2: return ET_E5M2;
        case ACL_FLOAT4_E2M1: return ET_E2M1;
        case ACL_FLOAT8_E8M0: return ET_E8M0;
        default: return ET_NONE;
    }
}
bool is_float_act(aclDataType t) { return t == ACL_FLOAT || t == ACL_FLOAT16 || t == ACL_BF16; }

// Path override for A/B measurements: B200_QMM_PATH=generic|gemv|tc (unset = automatic).
int forced_path() {
    const char *e = getenv("B200_QMM_PATH");
    if (!e) return -1;
    if (!strcmp(e, "generic")) return PATH_GENERIC;
    if (!strcmp(e, "gemv")) return PATH_GEMV;
    if (!strcmp(e, "tc")) return PATH_TC;
    return -1;
}
bool debug_on() {
    static const bool on = getenv("B200_QMM_DBG") != nullptr;
    return on;
}

const void *data_of(const aclTensor *t) {
    if (!t || !t->data) return nullptr;
    // Sub-byte tensors cannot carry an odd element offset; validated in phase 1.
    return (const char *)t->data + t->offset * (int64_t)elem_bits(elem_type(t->dtype)) / 8;
}

// MatmulArgs of a plan with the tensors' current data pointers.
MatmulArgs args_of(const aclOpExecutor *e, void *ws, uint64_t ws_bytes) {
    MatmulArgs p;
    p.a = data_of(e->a); p.b = data_of(e->b); p.out = const_cast<void *>(data_of(e->out));
    p.a_type = elem_type(e->a->dtype); p.b_type = elem_type(e->b->dtype); p.out_type = elem_type(e->out->dtype);
    p.batch = e->batch; p.M = e->m; p.N = e->n; p.K = e->k; p.group = e->group;
    p.a_batch_stride = e->m * e->k; p.b_batch_stride = e->k * e->n; p.out_batch_stride = e->m * e->n;
    p.b_transposed = e->b_transposed; p.accumulate = e->accumulate;
    p.b_nz = e->b->format == ACL_FORMAT_FRACTAL_NZ &&
             ((e->op == PLAN_WQBMM && e->b->dtype == ACL_INT4) || (e->op == PLAN_MX && e->b->dtype == ACL_FLOAT4_E2M1));
    p.split_k = e->split_k; p.workspace = ws; p.workspace_bytes = ws_bytes;
    if (e->bias) { p.bias = data_of(e->bias); p.bias_type = elem_type(e->bias->dtype); }
    switch (e->op) {
        case PLAN_WQBMM:
            p.epilogue = EPI_PLAIN;
            p.scale = data_of(e->scale); p.sc_type = elem_type(e->scale->dtype);
            p.offset = e->scale2 ? data_of(e->scale2) : nullptr;
            break;
        case PLAN_QMM:
            if (e->scale) {
                p.epilogue = EPI_DEQ_I32;
                p.scale = data_of(e->scale); p.sc_type = elem_type(e->scale->dtype);
                p.pertoken = e->pertoken ? (const float *)data_of(e->pertoken) : nullptr;
            } else {
                p.epilogue = EPI_RAW_I32;
            }
            break;
        case PLAN_MX:
            p.epilogue = EPI_PLAIN;
            p.a_scale = (const uint8_t *)data_of(e->scale);
            p.b_scale = (const uint8_t *)data_of(e->scale2);
            break;
        default: break;
    }
    return p;
}

// MatmulArgs for planning: every tensor that is present gets the same well-aligned stand-in address,
// so the plan (kernel family, split, workspace bytes) depends on presence, types and shapes only and a
// caller may hand over the data pointers later (aclSetRawTensorAddr between the phases).  If the real
// pointers then miss the alignment the planned kernel needs, phase 2 runs the generic kernel instead.
MatmulArgs plan_args_of(const aclOpExecutor *e) {
    MatmulArgs p = args_of(e, nullptr, 0);
    void *const here = reinterpret_cast<void *>(uintptr_t(1) << 20);
    p.a = p.b = p.out = here;
    if (e->bias) p.bias = here;
    switch (e->op) {
        case PLAN_WQBMM: p.scale = here; p.offset = e->scale2 ? here : nullptr; break;
        case PLAN_QMM: if (e->scale) { p.scale = here; p.pertoken = e->pertoken ? (const float *)here : nullptr; } break;
        case PLAN_MX: p.a_scale = p.b_scale = (const uint8_t *)here; break;
        default: break;
    }
    return p;
}

// Chooses the kernel family for a plan and sizes its workspace.
void choose_path(aclOpExecutor *e, uint64_t *ws) {
    MatmulArgs p = plan_args_of(e);
    int want = forced_path();
    e->path = PATH_GENERIC; e->split_k = 1; e->ws_bytes = 0;
    const bool tc_ok = tc_supported(p), gemv_ok = !p.b_nz && gemv_supported(p);
    if (p.b_nz) want = PATH_TC;   // only the tensor-core family reads the tile-packed weight layout
    if (want == PATH_TC && tc_ok) e->path = PATH_TC;
    else if (want == PATH_GEMV && gemv_ok) e->path = PATH_GEMV;
    else if (want == PATH_GENERIC) e->path = PATH_GENERIC;
    else if (tc_ok) e->path = PATH_TC;
    else if (gemv_ok) e->path = PATH_GEMV;
    if (e->path == PATH_GEMV) {
        p.split_k = e->split_k = gemv_pick_split_k(p);
        e->ws_bytes = gemv_workspace_bytes(p);
    } else if (e->path == PATH_TC) {
        tc_plan(p);
        e->split_k = p.split_k;
        e->ws_bytes = tc_workspace_bytes(p);
    }
    *ws = e->ws_bytes;
    if (debug_on())
        fprintf(stderr, "[b200-qmm] op=%d M=%ld N=%ld K=%ld group=%ld path=%d split_k=%d ws=%lu\n", (int)e->op, (long)e->m,
                (long)e->n, (long)e->k, (long)e->group, (int)e->path, e->split_k, (unsigned long)e->ws_bytes);
}

// Per device: the code of a bounded wait that gave up, as last seen by aclnnB200DeviceStatus().  While it is set the
// matmul entry points refuse to launch (361001): the results of the launch that gave up are undefined, and the
// application is expected to find out why before it goes on (aclnnB200ResetDeviceStatus() clears it).
std::atomic<uint32_t> g_latched_status[64];

uint32_t latched_status_of_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    return g_latched_status[dev].load(std::memory_order_relaxed);
}

aclnnStatus run_matmul(void *ws, uint64_t ws_bytes, aclOpExecutor *e, aclrtStream stream) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    aclnnStatus st = ACLNN_SUCCESS;
    if (const uint32_t code = latched_status_of_current_device()) {
        fprintf(stderr, "[b200-qmm] refusing to launch: an earlier kernel on this device gave up a bounded wait (code 0x%x); "
                        "call aclnnB200ResetDeviceStatus() once the cause is understood\n", code);
        st = ACLNN_ERR_RUNTIME_ERROR;
    } else if (e->op != PLAN_WQBMM && e->op != PLAN_QMM && e->op != PLAN_MX) {
        st = ACLNN_ERR_PARAM_INVALID;   // a plan of another operator (or of a composite one) was handed in
    } else if (e->m == 0 || e->n == 0) {
        // empty output: nothing to launch
    } else if (e->ws_bytes > 0 && (!ws || ws_bytes < e->ws_bytes)) {
        st = ACLNN_ERR_PARAM_INVALID;  // undersized workspace is rejected before anything is launched
    } else {
        MatmulArgs p = args_of(e, ws, ws_bytes);
        const bool scales_missing = (e->op == PLAN_WQBMM && (!p.scale || (e->scale2 && !p.offset))) ||
                                    (e->op == PLAN_QMM && e->scale && (!p.scale || (e->pertoken && !p.pertoken))) ||
                                    (e->op == PLAN_MX && (!p.a_scale || !p.b_scale)) || (e->bias && !p.bias);
        if (!p.a || !p.b || !p.out || scales_missing) st = ACLNN_ERR_PARAM_NULLPTR;
        else {
            cudaStream_t s = (cudaStream_t)stream;
            cudaError_t err;
            switch (e->path) {
                case PATH_GEMV: err = launch_gemv(p, s); break;
                case PATH_TC: err = launch_tc(p, s); break;
                default: err = launch_generic(p, s); break;
            }
            // The fast kernels refuse pointers off their load/store alignment before launching anything;
            // the bounds-checked generic kernel takes any address and needs no workspace.
            if (err == cudaErrorMisalignedAddress && e->path != PATH_GENERIC) err = launch_generic(p, s);
            if (err != cudaSuccess) {
                fprintf(stderr, "[b200-qmm] launch failed: %s\n", cudaGetErrorString(err));
                st = ACLNN_ERR_RUNTIME_ERROR;
            }
        }
    }
    delete e;
    return st;
}

bool shape_is(const aclTensor *t, std::initializer_list<int64_t> dims) {
    if (t->viewDims.size() != dims.size()) return false;
    size_t i = 0;
    for (auto d : dims) if (t->viewDims[i++] != d) return false;
    return true;
}
bool dense(const aclTensor *t) { return t->contiguous(); }

// ---- weight-only quantized matmul ------------------------------------------------------------------
aclnnStatus wqbmm_plan(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, const aclTensor *offset,
                       const aclTensor *bias, int64_t groupSize, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!x || !weight || !scale || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!is_float_act(x->dtype) || out->dtype != x->dtype) return ACLNN_ERR_PARAM_INVALID;
    if (weight->dtype != ACL_INT8 && weight->dtype != ACL_INT4) return ACLNN_ERR_PARAM_INVALID;
    if (scale->dtype != x->dtype || (offset && offset->dtype != x->dtype) || (bias && bias->dtype != x->dtype))
        return ACLNN_ERR_PARAM_INVALID;
    if (x->rank() != 2 || weight->rank() != 2 || out->rank() != 2) return ACLNN_ERR_PARAM_INVALID;
    const int64_t M = x->viewDims[0], K = x->viewDims[1], N = weight->viewDims[1];
    if (weight->viewDims[0] != K || !shape_is(out, {M, N}) || K <= 0 || N <= 0 || M < 0) return ACLNN_ERR_PARAM_INVALID;
    int64_t G = 1;
    if (scale->rank() == 1) { if (scale->viewDims[0] != N) return ACLNN_ERR_PARAM_INVALID; }
    else if (scale->rank() == 2) { G = scale->viewDims[0]; if (scale->viewDims[1] != N || G <= 0 || K % G != 0) return ACLNN_ERR_PARAM_INVALID; }
    else return ACLNN_ERR_PARAM_INVALID;
    if (offset && offset->viewDims != scale->viewDims) return ACLNN_ERR_PARAM_INVALID;
    if (bias && !shape_is(bias, {N})) return ACLNN_ERR_PARAM_INVALID;
    if (groupSize < 0 || (groupSize > 0 && G > 1 && groupSize != K / G)) return ACLNN_ERR_PARAM_INVALID;
    if (groupSize > 0 && G == 1 && groupSize < K) return ACLNN_ERR_PARAM_INVALID;
    if (weight->dtype == ACL_INT4 && (((K * N) & 1) || (weight->offset & 1))) return ACLNN_ERR_PARAM_INVALID;
    for (const aclTensor *t : {x, weight, scale, offset, bias, (const aclTensor *)out})
        if (t && !dense(t)) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new (std::nothrow) aclOpExecutor();
    if (!e) return ACLNN_ERR_RUNTIME_ERROR;
    e->op = PLAN_WQBMM; e->a = x; e->b = weight; e->scale = scale; e->scale2 = offset; e->bias = bias; e->out = out;
    e->m = M; e->n = N; e->k = K; e->group = K / G;
    choose_path(e, ws);
    if (weight->format == ACL_FORMAT_FRACTAL_NZ && weight->dtype == ACL_INT4 && e->path != PATH_TC) {
        // tile-packed int4 weights and a shape (or a device) the tensor-core family does not take
        delete e;
        return ACLNN_ERR_PARAM_INVALID;
    }
    *ex = e;
    return ACLNN_SUCCESS;
}

// ---- W8A8 quantized matmul -------------------------------------------------------------------------
struct QmmOpts { bool transposed = false, accumulate = false, batched = false; };

aclnnStatus qmm_plan(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, const aclTensor *pertoken,
                     const aclTensor *bias, aclTensor *out, QmmOpts o, uint64_t *ws, aclOpExecutor **ex) {
    if (!x || !weight || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!scale && out->dtype != ACL_INT32) return ACLNN_ERR_PARAM_NULLPTR;
    if (x->dtype != ACL_INT8 || weight->dtype != ACL_INT8) return ACLNN_ERR_PARAM_INVALID;
    if (scale && (!is_float_act(scale->dtype) || !is_float_act(out->dtype))) return ACLNN_ERR_PARAM_INVALID;
    if (!scale && (pertoken || o.accumulate)) return ACLNN_ERR_PARAM_INVALID;
    if (pertoken && pertoken->dtype != ACL_FLOAT) return ACLNN_ERR_PARAM_INVALID;
    if (bias && bias->dtype != ACL_INT32) return ACLNN_ERR_PARAM_INVALID;
    int64_t B = 1, M, K, N;
    if (o.batched) {
        if (x->rank() != 3 || weight->rank() != 3 || out->rank() != 3) return ACLNN_ERR_PARAM_INVALID;
        B = x->viewDims[0]; M = x->viewDims[1]; K = x->viewDims[2]; N = weight->viewDims[2];
        if (weight->viewDims[0] != B || weight->viewDims[1] != K || !shape_is(out, {B, M, N})) return ACLNN_ERR_PARAM_INVALID;
    } else {
        if (x->rank() != 2 || weight->rank() != 2 || out->rank() != 2) return ACLNN_ERR_PARAM_INVALID;
        M = x->viewDims[0]; K = x->viewDims[1];
        N = o.transposed ? weight->viewDims[0] : weight->viewDims[1];
        if ((o.transposed ? weight->viewDims[1] : weight->viewDims[0]) != K || !shape_is(out, {M, N})) return ACLNN_ERR_PARAM_INVALID;
    }
    if (K <= 0 || N <= 0 || M < 0 || B <= 0) return ACLNN_ERR_PARAM_INVALID;
    if (scale && !shape_is(scale, {N})) return ACLNN_ERR_PARAM_INVALID;
    if (pertoken && !shape_is(pertoken, {M})) return ACLNN_ERR_PARAM_INVALID;
    if (bias && !shape_is(bias, {N})) return ACLNN_ERR_PARAM_INVALID;
    // int32 accumulation is exact while K * 128 * 128 stays below 2^31.
    if (K > 131071) return ACLNN_ERR_PARAM_INVALID;
    for (const aclTensor *t : {x, weight, scale, pertoken, bias, (const aclTensor *)out})
        if (t && !dense(t)) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new (std::nothrow) aclOpExecutor();
    if (!e) return ACLNN_ERR_RUNTIME_ERROR;
    e->op = PLAN_QMM; e->a = x; e->b = weight; e->scale = scale; e->pertoken = pertoken; e->bias = bias; e->out = out;
    e->batch = B; e->m = M; e->n = N; e->k = K; e->group = K;
    e->b_transposed = o.transposed; e->accumulate = o.accumulate;
    choose_path(e, ws);
    *ex = e;
    return ACLNN_SUCCESS;
}

// ---- MX block-scaled matmul ------------------------------------------------------------------------
bool is_mx_operand(aclDataType t) { return t == ACL_FLOAT8_E4M3FN || t == ACL_FLOAT8_E5M2 || t == ACL_FLOAT4_E2M1; }

aclnnStatus mx_plan(const aclTensor *self, const aclTensor *selfScale, const aclTensor *other, const aclTensor *otherScale,
                    aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!self || !selfScale || !other || !otherScale || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!is_mx_operand(self->dtype) || !is_mx_operand(other->dtype)) return ACLNN_ERR_PARAM_INVALID;
    if (selfScale->dtype != ACL_FLOAT8_E8M0 || otherScale->dtype != ACL_FLOAT8_E8M0) return ACLNN_ERR_PARAM_INVALID;
    if (!is_float_act(out->dtype)) return ACLNN_ERR_PARAM_INVALID;
    if (self->rank() != 2 || other->rank() != 2 || out->rank() != 2) return ACLNN_ERR_PARAM_INVALID;
    const int64_t M = self->viewDims[0], K = self->viewDims[1], N = other->viewDims[1];
    if (other->viewDims[0] != K || !shape_is(out, {M, N}) || K <= 0 || N <= 0 || M < 0) return ACLNN_ERR_PARAM_INVALID;
    if (K % 32 != 0) return ACLNN_ERR_PARAM_INVALID;
    if (!shape_is(selfScale, {M, K / 32}) || !shape_is(otherScale, {K / 32, N})) return ACLNN_ERR_PARAM_INVALID;
    if (other->dtype == ACL_FLOAT4_E2M1 && (N & 1)) return ACLNN_ERR_PARAM_INVALID;
    if ((self->dtype == ACL_FLOAT4_E2M1 && (self->offset & 1)) || (other->dtype == ACL_FLOAT4_E2M1 && (other->offset & 1)))
        return ACLNN_ERR_PARAM_INVALID;
    for (const aclTensor *t : {self, selfScale, other, otherScale, (const aclTensor *)out})
        if (!dense(t)) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new (std::nothrow) aclOpExecutor();
    if (!e) return ACLNN_ERR_RUNTIME_ERROR;
    e->op = PLAN_MX; e->a = self; e->b = other; e->scale = selfScale; e->scale2 = otherScale; e->out = out;
    e->m = M; e->n = N; e->k = K; e->group = 32;
    choose_path(e, ws);
    if (other->format == ACL_FORMAT_FRACTAL_NZ && other->dtype == ACL_FLOAT4_E2M1 &&
        (e->path != PATH_TC || !mx_native_supported(plan_args_of(e)))) {
        delete e;   // widened fp4 weights are read by the native block-scaled kernel only
        return ACLNN_ERR_PARAM_INVALID;
    }
    *ex = e;
    return ACLNN_SUCCESS;
}

aclnnStatus run_simple(aclOpExecutor *e, aclrtStream stream) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t err = cudaSuccess;
    switch (e->op) {
        case PLAN_INT4_PACK:
            err = launch_int4_pack((const int8_t *)data_of(e->a), (uint8_t *)const_cast<void *>(data_of(e->out)), e->n, s);
            break;
        case PLAN_PACK_NZ:
            err = launch_wq_pack_nz(data_of(e->a), const_cast<void *>(data_of(e->out)), e->k, e->n, s);
            break;
        case PLAN_WIDEN_FP4:
            err = launch_mx_widen_fp4(data_of(e->a), const_cast<void *>(data_of(e->out)), e->n, s);
            break;
        case PLAN_COPY:
            err = cudaMemcpyAsync(const_cast<void *>(data_of(e->out)), data_of(e->a), (size_t)e->n, cudaMemcpyDeviceToDevice, s);
            break;
        case PLAN_WEIGHT_SIZE:
            err = launch_fill_i64((int64_t *)const_cast<void *>(data_of(e->out)), e->n, s);
            break;
        case PLAN_CAST:
            err = launch_cast(data_of(e->a), elem_type(e->a->dtype), const_cast<void *>(data_of(e->out)), elem_type(e->cast_to),
                              e->n, s);
            break;
        case PLAN_DYNQUANT:
            err = launch_dynamic_quant(data_of(e->a), elem_type(e->a->dtype), (int8_t *)const_cast<void *>(data_of(e->out)),
                                       (float *)const_cast<void *>(data_of(e->out2)), e->m, e->k, s);
            break;
        case PLAN_SWIGLUQUANT:
            err = launch_swiglu_quant(data_of(e->a), elem_type(e->a->dtype), e->pertoken ? (const float *)data_of(e->pertoken) : nullptr,
                                      (int8_t *)const_cast<void *>(data_of(e->out)),
                                      (float *)const_cast<void *>(data_of(e->out2)), e->m, e->k, s);
            break;
        case PLAN_MXQUANT:
            err = launch_dynamic_mx_quant(data_of(e->a), elem_type(e->a->dtype), (int8_t *)const_cast<void *>(data_of(e->out)),
                                          (float *)const_cast<void *>(data_of(e->out2)), e->m, e->k, s);
            break;
        case PLAN_ADDRMSNORM:
            err = launch_add_rmsnorm(data_of(e->a), data_of(e->b), e->scale ? data_of(e->scale) : nullptr, elem_type(e->a->dtype),
                                     e->scale ? elem_type(e->scale->dtype) : ET_NONE, const_cast<void *>(data_of(e->out2)),
                                     const_cast<void *>(data_of(e->out)), e->m, e->k, (float)e->eps, s);
            break;
        case PLAN_QPARAM:
            err = launch_qparam((const float *)data_of(e->a), e->b ? (const float *)data_of(e->b) : nullptr,
                                (int64_t *)const_cast<void *>(data_of(e->out)), e->n, s);
            break;
        default: err = cudaErrorInvalidValue;
    }
    delete e;
    return err == cudaSuccess ? ACLNN_SUCCESS : ACLNN_ERR_RUNTIME_ERROR;
}

}  // namespace

extern "C" {

uint64_t aclnnB200KernelLaunchCount(void) { return qmm::launch_count(); }
uint32_t aclnnB200DeviceStatus(void) {
    const uint32_t v = qmm::tc_device_status();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return v;
    if (v) g_latched_status[dev].store(v, std::memory_order_relaxed);
    return v ? v : g_latched_status[dev].load(std::memory_order_relaxed);
}
void aclnnB200ReserveSms(int32_t sms) { tc_reserve_sms(sms); }
void aclnnB200SetDecodeGather(const aclnnB200DecodeGather *g) {
    static_assert(sizeof(aclnnB200DecodeGather) == sizeof(DecodeGather), "the public struct mirrors the kernel's");
    wq_mma_set_gather(reinterpret_cast<const DecodeGather *>(g));
}
int32_t aclnnB200DecodeGatherConsumed(void) { return wq_mma_gather_consumed() ? 1 : 0; }

void aclnnB200ResetDeviceStatus(void) {
    qmm::tc_device_status_reset();
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) g_latched_status[dev].store(0, std::memory_order_relaxed);
}

#define RUN_MATMUL(NAME) \
    aclnnStatus NAME(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return run_matmul(ws, wsz, e, s); }

#define WQBMM_ALIAS(NAME)                                                                                             \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *antiquantScale, \
                                       const aclTensor *antiquantOffset, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) { \
        return wqbmm_plan(x, weight, antiquantScale, antiquantOffset, nullptr, 0, out, ws, ex);                       \
    }                                                                                                                 \
    RUN_MATMUL(NAME)
WQBMM_ALIAS(aclnnWeightQuantBatchMatmul)
WQBMM_ALIAS(aclnnWeightQuantBatchMatmulV2)
WQBMM_ALIAS(aclnnWeightQuantBatchMatmulV3)
WQBMM_ALIAS(aclnnWeightQuantBatchMatmulNz)

aclnnStatus aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(const aclTensor *x, const aclTensor *weight,
        const aclTensor *antiquantScale, const aclTensor *antiquantOffsetOptional, const aclTensor *biasOptional,
        int64_t antiquantGroupSize, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    return wqbmm_plan(x, weight, antiquantScale, antiquantOffsetOptional, biasOptional, antiquantGroupSize, out, ws, ex);
}
RUN_MATMUL(aclnnWeightQuantBatchMatmulV2Ex)

#define QMM_ALIAS(NAME, OPTS)                                                                                        \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *scale,          \
                                       aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {                           \
        if (!scale) return ACLNN_ERR_PARAM_NULLPTR;                                                                  \
        return qmm_plan(x, weight, scale, nullptr, nullptr, out, OPTS, ws, ex);                                      \
    }                                                                                                                \
    RUN_MATMUL(NAME)
QMM_ALIAS(aclnnQuantMatmul, QmmOpts{})
QMM_ALIAS(aclnnQuantMatmulV2, QmmOpts{})
QMM_ALIAS(aclnnQuantMatmulV3, QmmOpts{})
QMM_ALIAS(aclnnQuantMatmulV4, QmmOpts{})
QMM_ALIAS(aclnnQuantMatmulV5, QmmOpts{})
QMM_ALIAS(aclnnQuantMatmulDequant, QmmOpts{})
QMM_ALIAS(aclnnQuantMatmulWeightNz, QmmOpts{})
QMM_ALIAS(aclnnFusedQuantMatmul, QmmOpts{})
QMM_ALIAS(aclnnFusedQuantMatmulWeightNz, QmmOpts{})
QMM_ALIAS(aclnnMatmulCompressDequant, QmmOpts{})
QMM_ALIAS(aclnnSparse4to2QuantMatmulWeightNz, QmmOpts{})
QMM_ALIAS(aclnnDualLevelQuantMatmulWeightNz, QmmOpts{})
QMM_ALIAS(aclnnQuantBatchMatmulInplaceAdd, (QmmOpts{false, true, false}))
QMM_ALIAS(aclnnTransposeQuantBatchMatMul, (QmmOpts{true, false, false}))
QMM_ALIAS(aclnnBatchMatmulQuant, (QmmOpts{false, false, true}))

// Grouped (mixture-of-experts) forms.  With a 2-D weight [K,N] the group list is accepted and not used -- one
// group spanning every row -- exactly like the reference's placeholder (cuda/src/ops/matmul.cu:1195-1202,
// 1402-1413).  With a 3-D weight [E,K,N] the group list is honoured: it holds E entries, either the rows per
// group or their running totals (both must end at M), the rows of group g are multiplied by weight[g] and
// dequantised with scale[g] (scale [E,N], or [N] shared by all groups).  Each group is planned as a W8A8 matmul
// of its own over views of the caller's tensors; the workspace is the largest any group needs (they run one
// after the other on the stream).
}  // extern "C"
namespace {
struct GroupedPlan {
    struct Child {
        aclTensor x, w, scale, out;
        aclOpExecutor *ex = nullptr;
    };
    const aclTensor *x = nullptr, *w = nullptr, *scale = nullptr;
    aclTensor *out = nullptr;
    std::vector<Child *> children;
    ~GroupedPlan() {
        for (Child *c : children) { delete c->ex; delete c; }
    }
};
void free_grouped(void *p) { delete static_cast<GroupedPlan *>(p); }

aclTensor view_of(const aclTensor *t, std::vector<int64_t> dims, int64_t elem_offset) {
    aclTensor v;
    v.viewDims = dims; v.storageDims = dims;
    v.strides.resize(dims.size());
    int64_t st = 1;
    for (int i = (int)dims.size() - 1; i >= 0; --i) { v.strides[i] = st; st *= dims[i]; }
    v.offset = t->offset + elem_offset; v.dtype = t->dtype; v.format = ACL_FORMAT_ND; v.data = t->data;
    return v;
}

aclnnStatus grouped_plan(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, const aclIntArray *groupList,
                         aclTensor *out, QmmOpts o, uint64_t *ws, aclOpExecutor **ex) {
    if (!x || !weight || !scale || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (weight->rank() != 3) return qmm_plan(x, weight, scale, nullptr, nullptr, out, o, ws, ex);
    if (!groupList || x->rank() != 2 || out->rank() != 2) return ACLNN_ERR_PARAM_INVALID;
    const int64_t E = weight->viewDims[0], K = weight->viewDims[1], N = weight->viewDims[2], M = x->viewDims[0];
    if ((int64_t)groupList->v.size() != E || E < 1 || x->viewDims[1] != K || !shape_is(out, {M, N})) return ACLNN_ERR_PARAM_INVALID;
    const bool per_group_scale = scale->rank() == 2;
    if (per_group_scale ? !shape_is(scale, {E, N}) : !shape_is(scale, {N})) return ACLNN_ERR_PARAM_INVALID;
    for (const aclTensor *t : {x, weight, scale, (const aclTensor *)out})
        if (!dense(t)) return ACLNN_ERR_PARAM_INVALID;
    // rows per group: counts (sum = M) or running totals (non-decreasing, last = M)
    std::vector<int64_t> rows(E);
    int64_t sum = 0;
    bool counts_ok = true, totals_ok = true;
    for (int64_t g = 0; g < E; ++g) {
        const int64_t v = groupList->v[g];
        if (v < 0) return ACLNN_ERR_PARAM_INVALID;
        sum += v;
        if (g > 0 && v < groupList->v[g - 1]) totals_ok = false;
    }
    counts_ok = sum == M;
    totals_ok = totals_ok && groupList->v[E - 1] == M;
    if (!counts_ok && !totals_ok) return ACLNN_ERR_PARAM_INVALID;
    for (int64_t g = 0; g < E; ++g) rows[g] = counts_ok ? groupList->v[g] : groupList->v[g] - (g ? groupList->v[g - 1] : 0);

    auto *plan = new GroupedPlan();
    plan->x = x; plan->w = weight; plan->scale = scale; plan->out = out;
    uint64_t need = 0;
    int64_t r0 = 0;
    for (int64_t g = 0; g < E; ++g) {
        if (rows[g] == 0) continue;
        auto *c = new GroupedPlan::Child();
        c->x = view_of(x, {rows[g], K}, r0 * K);
        c->w = view_of(weight, {K, N}, g * K * N);
        c->scale = view_of(scale, {N}, per_group_scale ? g * N : 0);
        c->out = view_of(out, {rows[g], N}, r0 * N);
        plan->children.push_back(c);
        uint64_t w1 = 0;
        const aclnnStatus st = qmm_plan(&c->x, &c->w, &c->scale, nullptr, nullptr, &c->out, o, &w1, &c->ex);
        if (st != ACLNN_SUCCESS) { delete plan; return st; }
        need = w1 > need ? w1 : need;
        r0 += rows[g];
    }
    auto *e = new (std::nothrow) aclOpExecutor();
    if (!e) { delete plan; return ACLNN_ERR_RUNTIME_ERROR; }
    e->op = PLAN_WRAPPER; e->payload = plan; e->payload_free = free_grouped;
    *ws = need; *ex = e;
    return ACLNN_SUCCESS;
}

aclnnStatus run_grouped(void *ws, uint64_t ws_bytes, aclOpExecutor *e, aclrtStream stream) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    if (e->op != PLAN_WRAPPER || e->payload_free != free_grouped) return run_matmul(ws, ws_bytes, e, stream);   // 2-D weight: one plain matmul
    auto *plan = static_cast<GroupedPlan *>(e->payload);
    aclnnStatus st = ACLNN_SUCCESS;
    for (GroupedPlan::Child *c : plan->children) {
        // the caller may have handed over the data pointers after phase 1
        c->x.data = plan->x->data; c->w.data = plan->w->data; c->scale.data = plan->scale->data; c->out.data = plan->out->data;
        aclOpExecutor *child = c->ex;
        c->ex = nullptr;   // run_matmul consumes it
        const aclnnStatus s1 = run_matmul(ws, ws_bytes, child, stream);
        if (s1 != ACLNN_SUCCESS && st == ACLNN_SUCCESS) st = s1;
    }
    delete e;
    return st;
}
}  // namespace
extern "C" {

#define QMM_GROUPED_ALIAS(NAME, OPTS)                                                                                \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *scale,          \
                                       const aclIntArray *groupList, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) { \
        return grouped_plan(x, weight, scale, groupList, out, OPTS, ws, ex);                                         \
    }                                                                                                                \
    aclnnStatus NAME(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return run_grouped(ws, wsz, e, s); }
QMM_GROUPED_ALIAS(aclnnQuantGroupedMatmulDequant, QmmOpts{})
QMM_GROUPED_ALIAS(aclnnQuantGroupedMatmulDequantWeightNZ, QmmOpts{})
QMM_GROUPED_ALIAS(aclnnQuantGroupedMatmulInplaceAdd, (QmmOpts{false, true, false}))

// Collective-signature names whose communicator the reference ignores (cuda/src/ops/matmul.cu:1294-1302):
// the local W8A8 matmul.
#define QMM_COMM_ALIAS(NAME)                                                                                         \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, void *comm, \
                                       aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {                           \
        (void)comm;                                                                                                  \
        if (!scale) return ACLNN_ERR_PARAM_NULLPTR;                                                                  \
        return qmm_plan(x, weight, scale, nullptr, nullptr, out, QmmOpts{}, ws, ex);                                 \
    }                                                                                                                \
    RUN_MATMUL(NAME)
QMM_COMM_ALIAS(aclnnAlltoAllQuantMatmul)
QMM_COMM_ALIAS(aclnnQuantMatmulAlltoAll)
QMM_COMM_ALIAS(aclnnAlltoAllvQuantGroupedMatMul)
QMM_COMM_ALIAS(aclnnQuantGroupedMatMulAlltoAllv)
QMM_COMM_ALIAS(aclnnQuantReduceScatter)
QMM_COMM_ALIAS(aclnnQuantMatmulReduceSumWeightNz)

aclnnStatus aclnnQuantMatmulV4ExGetWorkspaceSize(const aclTensor *x1, const aclTensor *x2, const aclTensor *scale,
        const aclTensor *offsetOptional, const aclTensor *pertokenScaleOptional, const aclTensor *biasOptional,
        aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (offsetOptional) return ACLNN_ERR_PARAM_INVALID;
    return qmm_plan(x1, x2, scale, pertokenScaleOptional, biasOptional, out, QmmOpts{}, ws, ex);
}
RUN_MATMUL(aclnnQuantMatmulV4Ex)

#define MX_ALIAS(NAME)                                                                                               \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *self, const aclTensor *selfScale, const aclTensor *other,    \
                                       const aclTensor *otherScale, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) { \
        return mx_plan(self, selfScale, other, otherScale, out, ws, ex);                                             \
    }                                                                                                                \
    RUN_MATMUL(NAME)
MX_ALIAS(aclnnMatmulMxFp8)
MX_ALIAS(aclnnMatmulMxFp8Hw)
MX_ALIAS(aclnnMatmulMxFp4)
MX_ALIAS(aclnnMatmulMxFp4Hw)

// Single-call decode matmul that allocates nothing and takes no workspace (see gemv.cu).
aclnnStatus aclnnB200WeightQuantMatmulNoAlloc(const void *x, const void *weight, const void *antiquantScale,
        const void *antiquantOffsetOptional, const void *biasOptional, void *out, int64_t m, int64_t k, int64_t n,
        int64_t antiquantGroupSize, aclDataType xType, aclDataType weightType, aclrtStream stream) {
    if (!x || !weight || !antiquantScale || !out) return ACLNN_ERR_PARAM_NULLPTR;
    if (m < 1 || k < 1 || n < 1 || antiquantGroupSize < 0) return ACLNN_ERR_PARAM_INVALID;
    if (antiquantGroupSize > 0 && k % antiquantGroupSize != 0) return ACLNN_ERR_PARAM_INVALID;
    MatmulArgs p;
    p.a = x; p.b = weight; p.out = out; p.scale = antiquantScale; p.offset = antiquantOffsetOptional; p.bias = biasOptional;
    p.a_type = p.out_type = p.sc_type = elem_type(xType);
    p.bias_type = biasOptional ? p.a_type : (int)ET_NONE;
    p.b_type = elem_type(weightType);
    p.epilogue = EPI_PLAIN;
    p.M = m; p.N = n; p.K = k;
    p.group = (antiquantGroupSize == 0 || antiquantGroupSize >= k) ? k : antiquantGroupSize;
    if (!gemv_supported(p)) {
        fprintf(stderr, "[b200-qmm] aclnnB200WeightQuantMatmulNoAlloc: unsupported problem (needs M <= %d, fp16/bf16/fp32 "
                        "activations, int8/int4 weights, N %% 32 == 0, K a multiple of the group size)\n", gemv_max_m());
        return ACLNN_ERR_PARAM_INVALID;
    }
    bool too_large = false;
    cudaError_t err = launch_gemv_noalloc(p, (cudaStream_t)stream, &too_large);
    if (too_large) {
        fprintf(stderr, "[b200-qmm] aclnnB200WeightQuantMatmulNoAlloc: M=%ld N=%ld K=%ld needs more than the %zu bytes of "
                        "built-in scratch; use aclnnWeightQuantBatchMatmulV2 with a workspace\n", (long)m, (long)n, (long)k,
                noalloc_scratch_bytes());
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (err != cudaSuccess) {
        fprintf(stderr, "[b200-qmm] aclnnB200WeightQuantMatmulNoAlloc: %s\n", cudaGetErrorString(err));
        return ACLNN_ERR_RUNTIME_ERROR;
    }
    return ACLNN_SUCCESS;
}

#define RUN_SIMPLE(NAME) \
    aclnnStatus NAME(void *, uint64_t, aclOpExecutor *e, aclrtStream s) { return run_simple(e, s); }

aclnnStatus aclnnConvertWeightToINT4PackGetWorkspaceSize(const aclTensor *weight, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!weight || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!weight->data || !out->data) return ACLNN_ERR_PARAM_NULLPTR;
    if (weight->dtype != ACL_INT8 || !dense(weight) || !dense(out)) return ACLNN_ERR_PARAM_INVALID;
    if (weight->numel() & 1) return ACLNN_ERR_PARAM_INVALID;
    // out holds numel/2 bytes: an int8/uint8 tensor of half the elements, or an ACL_INT4 tensor of all of them.
    const int64_t n_out = weight->numel() / 2;
    const int64_t out_bytes = out->dtype == ACL_INT4 ? out->numel() / 2 : out->numel() * (int64_t)dtype_size(out->dtype);
    if (out_bytes != n_out) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_INT4_PACK; e->a = weight; e->out = out; e->n = n_out;
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
RUN_SIMPLE(aclnnConvertWeightToINT4Pack)

// Elements a tensor's storage holds (the product of its storage dimensions; the view's when none were given).
static int64_t storage_elems(const aclTensor *t) {
    if (t->storageDims.empty()) return t->numel();
    int64_t n = 1;
    for (auto d : t->storageDims) n *= d;
    return n;
}

// One-time re-layout of a weight into the on-device format its `out` tensor names.  An int4 [K,N] weight
// into an ACL_FORMAT_FRACTAL_NZ tensor becomes the tile-packed layout the decode kernel streams with
// contiguous 16 KB copies (out keeps the view shape [K,N]; its storage must hold the element count
// aclnnCalculateMatmulWeightSizeV2 reports for ACL_INT4).  Everything else is an identity copy, as in the
// reference (cuda/src/ops/matmul.cu:1162-1165).
aclnnStatus aclnnTransMatmulWeightGetWorkspaceSize(const aclTensor *weight, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!weight || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!weight->data || !out->data) return ACLNN_ERR_PARAM_NULLPTR;
    if (weight->dtype != out->dtype || weight->numel() != out->numel() || !dense(weight) || !dense(out)) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->a = weight; e->out = out;
    if (out->format == ACL_FORMAT_FRACTAL_NZ && weight->dtype == ACL_INT4 && weight->format != ACL_FORMAT_FRACTAL_NZ) {
        if (weight->rank() != 2 || out->viewDims != weight->viewDims || (weight->viewDims[1] & 1) || (weight->offset & 1) || out->offset != 0 ||
            storage_elems(out) < (int64_t)(2 * wq_nz_bytes(weight->viewDims[0], weight->viewDims[1]))) {
            delete e;
            return ACLNN_ERR_PARAM_INVALID;
        }
        e->op = PLAN_PACK_NZ; e->k = weight->viewDims[0]; e->n = weight->viewDims[1];
    } else if (out->format == ACL_FORMAT_FRACTAL_NZ && weight->dtype == ACL_FLOAT4_E2M1 && weight->format != ACL_FORMAT_FRACTAL_NZ) {
        // fp4 weight of a block-scaled matmul: one byte per element, the fp8 e4m3 code of the same value
        if (weight->rank() != 2 || out->viewDims != weight->viewDims || (weight->numel() % 32) || (weight->offset & 1) || out->offset != 0 ||
            storage_elems(out) < 2 * weight->numel()) {
            delete e;
            return ACLNN_ERR_PARAM_INVALID;
        }
        e->op = PLAN_WIDEN_FP4; e->n = weight->numel();
    } else {
        e->op = PLAN_COPY;
        e->n = (weight->numel() * elem_bits(elem_type(weight->dtype)) + 7) / 8;
    }
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
RUN_SIMPLE(aclnnTransMatmulWeight)

// Element count of the on-device form of a weight of the given shape.  Without a type (or for any type but
// int4) that is the product of the dimensions, as in the reference (cuda/src/ops/matmul.cu:1166-1170); for
// ACL_INT4 [K,N] it is the element count of the tile-packed layout (K padded to 128, N to 256).
static aclnnStatus weight_size_plan(const aclIntArray *shape, int64_t dtype, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!shape || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!out->data) return ACLNN_ERR_PARAM_NULLPTR;
    if (out->dtype != ACL_INT64 || out->numel() < 1) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_WEIGHT_SIZE; e->out = out; e->n = 1;
    for (auto d : shape->v) e->n *= d;
    if (dtype == (int64_t)ACL_INT4 && shape->v.size() == 2 && shape->v[0] > 0 && shape->v[1] > 0)
        e->n = (int64_t)(2 * wq_nz_bytes(shape->v[0], shape->v[1]));
    if (dtype == (int64_t)ACL_FLOAT4_E2M1) e->n *= 2;   // widened to one byte per element = the storage of two packed ones
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
aclnnStatus aclnnCalculateMatmulWeightSizeGetWorkspaceSize(const aclIntArray *weightShape, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    return weight_size_plan(weightShape, -1, out, ws, ex);
}
RUN_SIMPLE(aclnnCalculateMatmulWeightSize)
aclnnStatus aclnnCalculateMatmulWeightSizeV2GetWorkspaceSize(const aclIntArray *weightShape, int64_t dtype, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    return weight_size_plan(weightShape, dtype, out, ws, ex);
}
RUN_SIMPLE(aclnnCalculateMatmulWeightSizeV2)

// Per-token dynamic int8 quantiser: x [..., D] -> int8 of the same shape + fp32 scale per row
// (cuda/src/ops/quant.cu:99-111; V2-V4 are the reference's version aliases).
static aclnnStatus dynquant_plan(const aclTensor *x, aclTensor *out, aclTensor *scaleOut, uint64_t *ws, aclOpExecutor **ex) {
    if (!x || !out || !scaleOut || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (x->viewDims.empty()) return ACLNN_ERR_PARAM_INVALID;
    if (x->numel() > 0 && (!x->data || !out->data || !scaleOut->data)) return ACLNN_ERR_PARAM_NULLPTR;
    if (out->dtype != ACL_INT8 || scaleOut->dtype != ACL_FLOAT || x->viewDims != out->viewDims) return ACLNN_ERR_PARAM_INVALID;
    if (x->dtype != ACL_FLOAT && x->dtype != ACL_FLOAT16 && x->dtype != ACL_BF16) return ACLNN_ERR_PARAM_INVALID;
    if (!dense(x) || !dense(out) || !dense(scaleOut)) return ACLNN_ERR_PARAM_INVALID;
    const int64_t D = x->viewDims.back();
    const int64_t rows = D > 0 ? x->numel() / D : 0;
    if (scaleOut->numel() != rows) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_DYNQUANT; e->a = x; e->out = out; e->out2 = scaleOut; e->m = rows; e->k = D;
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
#define DYNQUANT_ALIAS(NAME)                                                                                         \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, aclTensor *out, aclTensor *scaleOut, uint64_t *ws,        \
                                       aclOpExecutor **ex) { return dynquant_plan(x, out, scaleOut, ws, ex); }      \
    RUN_SIMPLE(NAME)
DYNQUANT_ALIAS(aclnnDynamicQuant)
DYNQUANT_ALIAS(aclnnDynamicQuantV2)
DYNQUANT_ALIAS(aclnnDynamicQuantV3)
DYNQUANT_ALIAS(aclnnDynamicQuantV4)

// Residual add + RMS norm (cuda/src/ops/norm_ext.cu:233-247): y = rmsnorm(x + residual) * gamma,
// residualSum = x + residual.  Needed here as the tail of the all-reduce matmuls.
aclnnStatus aclnnAddRmsNormGetWorkspaceSize(const aclTensor *x, const aclTensor *residual, const aclTensor *gamma, double eps,
                                            aclTensor *y, aclTensor *residualSum, uint64_t *ws, aclOpExecutor **ex) {
    if (!x || !residual || !y || !residualSum || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (x->numel() > 0 && (!x->data || !residual->data || !y->data || !residualSum->data || (gamma && !gamma->data)))
        return ACLNN_ERR_PARAM_NULLPTR;
    if (x->dtype != ACL_FLOAT && x->dtype != ACL_FLOAT16 && x->dtype != ACL_BF16) return ACLNN_ERR_PARAM_INVALID;
    if (residual->dtype != x->dtype || y->dtype != x->dtype || residualSum->dtype != x->dtype) return ACLNN_ERR_PARAM_INVALID;
    if (x->viewDims.empty() || x->viewDims != residual->viewDims || x->viewDims != y->viewDims || x->viewDims != residualSum->viewDims)
        return ACLNN_ERR_PARAM_INVALID;
    const int64_t D = x->viewDims.back();
    if (gamma) {
        if (gamma->dtype != ACL_FLOAT && gamma->dtype != ACL_FLOAT16 && gamma->dtype != ACL_BF16) return ACLNN_ERR_PARAM_INVALID;
        if (gamma->numel() != D || !dense(gamma)) return ACLNN_ERR_PARAM_INVALID;
    }
    if (!dense(x) || !dense(residual) || !dense(y) || !dense(residualSum)) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_ADDRMSNORM; e->a = x; e->b = residual; e->scale = gamma; e->out = y; e->out2 = residualSum;
    e->m = D > 0 ? x->numel() / D : 0; e->k = D; e->eps = eps;
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
RUN_SIMPLE(aclnnAddRmsNorm)

// SwiGLU fused with the per-token quantiser: x [..., 2 D] -> int8 [..., D] + fp32 scale per row
// (cuda/src/ops/glu_ext.cu:118-141; V2 is the reference's alias).
static aclnnStatus swigluquant_plan(const aclTensor *x, const aclTensor *dq, aclTensor *out, aclTensor *scaleOut, uint64_t *ws,
                                    aclOpExecutor **ex) {
    if (!x || !out || !scaleOut || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (x->viewDims.empty() || out->viewDims.size() != x->viewDims.size()) return ACLNN_ERR_PARAM_INVALID;
    if (x->numel() > 0 && (!x->data || !out->data || !scaleOut->data)) return ACLNN_ERR_PARAM_NULLPTR;
    if (out->dtype != ACL_INT8 || scaleOut->dtype != ACL_FLOAT) return ACLNN_ERR_PARAM_INVALID;
    if (x->dtype != ACL_FLOAT && x->dtype != ACL_FLOAT16 && x->dtype != ACL_BF16) return ACLNN_ERR_PARAM_INVALID;
    const int64_t D = out->viewDims.back();
    if (x->viewDims.back() != 2 * D) return ACLNN_ERR_PARAM_INVALID;
    for (size_t i = 0; i + 1 < x->viewDims.size(); ++i)
        if (x->viewDims[i] != out->viewDims[i]) return ACLNN_ERR_PARAM_INVALID;
    if (!dense(x) || !dense(out) || !dense(scaleOut)) return ACLNN_ERR_PARAM_INVALID;
    const int64_t rows = D > 0 ? out->numel() / D : 0;
    if (scaleOut->numel() != rows) return ACLNN_ERR_PARAM_INVALID;
    if (dq) {   // optional per-row dequant scale
        if (x->numel() > 0 && !dq->data) return ACLNN_ERR_PARAM_NULLPTR;
        if (dq->dtype != ACL_FLOAT || dq->numel() != rows || !dense(dq)) return ACLNN_ERR_PARAM_INVALID;
    }
    auto *e = new aclOpExecutor();
    e->op = PLAN_SWIGLUQUANT; e->a = x; e->pertoken = dq; e->out = out; e->out2 = scaleOut; e->m = rows; e->k = D;
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
#define SWIGLUQUANT_ALIAS(NAME)                                                                                      \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, aclTensor *out, aclTensor *scaleOut, uint64_t *ws,        \
                                       aclOpExecutor **ex) { return swigluquant_plan(x, nullptr, out, scaleOut, ws, ex); } \
    RUN_SIMPLE(NAME)
SWIGLUQUANT_ALIAS(aclnnSwiGluQuant)
SWIGLUQUANT_ALIAS(aclnnSwiGluQuantV2)
// The same behind a per-row dequant scale: a and b are multiplied by dequantScale[row] first
// (cuda/src/ops/norm_ext.cu:1354-1369,1416-1432; V2 is the reference's alias).
#define DEQSWIGLUQUANT_ALIAS(NAME)                                                                                   \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *dequantScale, aclTensor *out, aclTensor *scaleOut, \
                                       uint64_t *ws, aclOpExecutor **ex) {                                           \
        return swigluquant_plan(x, dequantScale, out, scaleOut, ws, ex);                                             \
    }                                                                                                                \
    RUN_SIMPLE(NAME)
DEQSWIGLUQUANT_ALIAS(aclnnDequantSwigluQuant)
DEQSWIGLUQUANT_ALIAS(aclnnDequantSwigluQuantV2)

// Block-wise int8 quantiser with power-of-two scales (cuda/src/ops/quant.cu:380-389,496-514).
static aclnnStatus mxquant_plan(const aclTensor *x, int64_t blockSize, aclTensor *out, aclTensor *scaleOut, uint64_t *ws,
                                aclOpExecutor **ex) {
    if (!x || !out || !scaleOut || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (blockSize <= 0) return ACLNN_ERR_PARAM_INVALID;
    if (x->numel() > 0 && (!x->data || !out->data || !scaleOut->data)) return ACLNN_ERR_PARAM_NULLPTR;
    if (out->dtype != ACL_INT8 || scaleOut->dtype != ACL_FLOAT || x->viewDims != out->viewDims) return ACLNN_ERR_PARAM_INVALID;
    if (x->dtype != ACL_FLOAT && x->dtype != ACL_FLOAT16 && x->dtype != ACL_BF16) return ACLNN_ERR_PARAM_INVALID;
    if (x->numel() % blockSize != 0 || scaleOut->numel() != x->numel() / blockSize) return ACLNN_ERR_PARAM_INVALID;
    if (!dense(x) || !dense(out) || !dense(scaleOut)) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_MXQUANT; e->a = x; e->out = out; e->out2 = scaleOut; e->m = x->numel() / blockSize; e->k = blockSize;
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
#define MXQUANT_ALIAS(NAME)                                                                                          \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, int64_t blockSize, aclTensor *out, aclTensor *scaleOut,   \
                                       uint64_t *ws, aclOpExecutor **ex) { return mxquant_plan(x, blockSize, out, scaleOut, ws, ex); } \
    RUN_SIMPLE(NAME)
MXQUANT_ALIAS(aclnnDynamicMxQuant)
MXQUANT_ALIAS(aclnnDynamicMxQuantV2)

// fp32 scale (+ optional fp32 offset) -> int64 quant parameter (cuda/src/ops/quant.cu:657-673).
static aclnnStatus qparam_plan(const aclTensor *scale, const aclTensor *offset, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!scale || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (!scale->data || !out->data || (offset && !offset->data)) return ACLNN_ERR_PARAM_NULLPTR;
    if (scale->dtype != ACL_FLOAT || out->dtype != ACL_INT64 || (offset && offset->dtype != ACL_FLOAT)) return ACLNN_ERR_PARAM_INVALID;
    if (scale->numel() != out->numel() || (offset && offset->numel() != out->numel())) return ACLNN_ERR_PARAM_INVALID;
    if (!dense(scale) || !dense(out) || (offset && !dense(offset))) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_QPARAM; e->a = scale; e->b = offset; e->out = out; e->n = out->numel();
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
#define QPARAM_ALIAS(NAME)                                                                                           \
    aclnnStatus NAME##GetWorkspaceSize(const aclTensor *scale, const aclTensor *offset, aclTensor *out, uint64_t *ws, \
                                       aclOpExecutor **ex) { return qparam_plan(scale, offset, out, ws, ex); }       \
    RUN_SIMPLE(NAME)
QPARAM_ALIAS(aclnnTransQuantParam)
QPARAM_ALIAS(aclnnTransQuantParamV2)
QPARAM_ALIAS(aclnnTransQuantParamV3)

aclnnStatus aclnnCastGetWorkspaceSize(const aclTensor *self, aclDataType dtype, aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    if (!self || !out || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    if (out->dtype != dtype || self->viewDims != out->viewDims) return ACLNN_ERR_PARAM_INVALID;
    if (!dense(self) || !dense(out)) return ACLNN_ERR_PARAM_INVALID;
    const int st = elem_type(self->dtype), dt = elem_type(dtype);
    if (st == ET_NONE || dt == ET_NONE || st == ET_I4 || dt == ET_I4 || dt == ET_E8M0) return ACLNN_ERR_PARAM_INVALID;
    auto *e = new aclOpExecutor();
    e->op = PLAN_CAST; e->a = self; e->out = out; e->cast_to = dtype; e->n = self->numel();
    *ws = 0; *ex = e;
    return ACLNN_SUCCESS;
}
RUN_SIMPLE(aclnnCast)

}  // extern "C"
