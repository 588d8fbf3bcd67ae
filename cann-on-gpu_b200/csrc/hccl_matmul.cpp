// Quantized matmuls followed by an all-reduce over a communicator (K-split tensor parallelism): the
// local operator of libascendcl.so, then HcclAllReduce(SUM) of the output on the caller's stream.
// Scales are linear over the K reduction, so summing the ranks' scaled partial outputs equals
// scaling the full sum.  comm == NULL gives the local result (exact for one rank).
//
// Same contract as the reference's cuda/src/ops/mc2_ext.cu:67-87,185-195 and
// cuda/src/ops/matmul.cu:1304-1319, but the state travels in the executor handed back to the
// caller instead of a process-wide map (the reference's maps are not thread-safe).
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <mutex>

#include "aclnnop/aclnn_quant_matmul_mc2.h"
#include "hccl_p2p.h"

namespace {

// What phase 2 needs: the local operator's executor and what to all-reduce afterwards.  It rides in a
// wrapper plan of libascendcl.so, which owns it: destroying the plan (a caller that gives up after
// phase 1) ends up in free_allreduce.
struct AllReduceExecutor {
    aclOpExecutor *inner = nullptr;
    HcclComm comm = nullptr;
    const aclTensor *x = nullptr, *weight = nullptr, *scale = nullptr, *offset = nullptr;
    const aclTensor *out = nullptr;
    bool weight_only = false;
    int chunks = 1;          // row chunks whose all-reduce overlaps the next chunk's matmul
    int64_t rows = 0;
};
std::atomic<uint64_t> g_fused_allreduces{0};   // all-reduce matmuls that took the fused form (diagnostics)
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

// ---- overlap of the all-reduce with the matmul ---------------------------------------------------
// On request the output is produced in row chunks (contiguous in the [M,N] output): the all-reduce of
// chunk i runs on a second stream, behind an event, while the matmul of chunk i+1 runs on the caller's
// stream, which waits for the last all-reduce at the end.  The reference runs the whole matmul and then
// the whole all-reduce on one stream (cuda/src/ops/mc2_ext.cu:79-87).
// The second stream and the events belong to the communicator and live as long as the process.
constexpr int MAX_CHUNKS = 8;
struct OverlapLane {
    aclrtStream stream = nullptr;
    aclrtEvent ready[MAX_CHUNKS] = {};
    aclrtEvent done = nullptr;
};
std::mutex g_lane_mutex;
std::map<HcclComm, OverlapLane> g_lanes;

OverlapLane *lane_of(HcclComm comm) {
    std::lock_guard<std::mutex> lock(g_lane_mutex);
    auto it = g_lanes.find(comm);
    if (it != g_lanes.end()) return &it->second;
    OverlapLane l;
    if (aclrtCreateStream(&l.stream) != ACL_SUCCESS) return nullptr;
    bool ok = aclrtCreateEvent(&l.done) == ACL_SUCCESS;
    for (int i = 0; ok && i < MAX_CHUNKS; ++i) ok = aclrtCreateEvent(&l.ready[i]) == ACL_SUCCESS;
    if (!ok) return nullptr;
    return &g_lanes.emplace(comm, l).first->second;
}

// Row chunks for a matmul of `rows` rows.  Off unless asked for (B200_HCCL_OVERLAP_CHUNKS=<n>, at most eight): on
// two B200s the chunked form measured slower than the plain sequence at every setting tried (W8A8 4096 x 4096 x 14336,
// bf16 out: 370 us plain; 398-416 us with two or four chunks and 0-32 SMs left to the all-reduce) -- the all-reduce
// of the 117 MB output takes 250 us alone, 2.5 times the matmul, runs less efficiently in four pieces, and shares
// HBM bandwidth with the matmul beside it.
int chunks_for(int64_t rows) {
    int c = 1;
    if (const char *e = getenv("B200_HCCL_OVERLAP_CHUNKS")) c = atoi(e);
    if (c < 1) c = 1;
    if (c > MAX_CHUNKS) c = MAX_CHUNKS;
    if (c > rows / 16) c = rows >= 16 ? (int)(rows / 16) : 1;
    return c;
}
// SMs the chunked matmuls leave to the all-reduce kernels that run beside them (B200_HCCL_OVERLAP_SMS, default 20).
int overlap_sms() {
    if (const char *e = getenv("B200_HCCL_OVERLAP_SMS")) return atoi(e) > 0 ? atoi(e) : 0;
    return 20;
}
struct SmReservation {
    explicit SmReservation(int n) { aclnnB200ReserveSms(n); }
    ~SmReservation() { aclnnB200ReserveSms(0); }
};
int64_t chunk_begin(int64_t rows, int chunks, int i) { return rows * i / chunks / 16 * 16; }   // chunk edges on multiples of 16 rows

aclnnStatus local_plan(bool weight_only, const aclTensor *x, const aclTensor *weight, const aclTensor *scale, const aclTensor *offset,
                       const aclTensor *out, uint64_t *ws, aclOpExecutor **ex) {
    return weight_only ? aclnnWeightQuantBatchMatmulGetWorkspaceSize(x, weight, scale, offset, const_cast<aclTensor *>(out), ws, ex)
                       : aclnnQuantMatmulGetWorkspaceSize(x, weight, scale, const_cast<aclTensor *>(out), ws, ex);
}

aclnnStatus wrap(aclnnStatus st, aclOpExecutor *inner, HcclComm comm, const aclTensor *x, const aclTensor *weight, const aclTensor *scale,
                 const aclTensor *offset, const aclTensor *out, bool weight_only, uint64_t *ws, aclOpExecutor **ex) {
    if (st != ACLNN_SUCCESS) return st;
    aclDataType dt;
    HcclDataType ht;
    if (aclGetDataType(out, &dt) != ACLNN_SUCCESS || (comm && !hccl_type(dt, &ht))) {
        aclDestroyAclOpExecutor(inner);
        return ACLNN_ERR_PARAM_INVALID;
    }
    auto *w = new AllReduceExecutor();
    w->inner = inner; w->comm = comm; w->x = x; w->weight = weight; w->scale = scale; w->offset = offset; w->out = out;
    w->weight_only = weight_only;
    // chunked form: two-dimensional activations and output only; the workspace must serve the largest chunk too
    int64_t *xd = nullptr, *od = nullptr;
    uint64_t xn = 0, on = 0;
    if (comm && aclGetViewShape(x, &xd, &xn) == ACLNN_SUCCESS && aclGetViewShape(out, &od, &on) == ACLNN_SUCCESS && xn == 2 && on == 2 &&
        xd[0] == od[0]) {
        w->rows = xd[0];
        w->chunks = chunks_for(w->rows);
        if (w->chunks > 1) {
            // every chunk height is planned once here so that the workspace serves each of them
            SmReservation reserve(overlap_sms());
            int64_t seen_height = -1;
            for (int i = 0; i < w->chunks && w->chunks > 1; ++i) {
                const int64_t r0 = chunk_begin(w->rows, w->chunks, i), r1 = i + 1 == w->chunks ? w->rows : chunk_begin(w->rows, w->chunks, i + 1);
                if (r1 <= r0 || r1 - r0 == seen_height) continue;
                seen_height = r1 - r0;
                aclTensor *xs = aclnnB200CreateRowSlice(x, r0, r1 - r0), *os = aclnnB200CreateRowSlice(out, r0, r1 - r0);
                uint64_t need = 0;
                aclOpExecutor *probe = nullptr;
                if (xs && os && local_plan(weight_only, xs, weight, scale, offset, os, &need, &probe) == ACLNN_SUCCESS) {
                    aclDestroyAclOpExecutor(probe);
                    if (need > *ws) *ws = need;
                } else {
                    w->chunks = 1;   // a chunk the local operator does not take: the plain sequence
                }
                if (xs) aclDestroyTensor(xs);
                if (os) aclDestroyTensor(os);
            }
        }
    }
    // the weight-only decode kernel can send its partial result to the peers itself (run below): its plan may need a
    // different workspace, and which form phase 2 takes is known only there
    if (comm && weight_only) {
        aclnnB200DecodeGather fake{};
        fake.nranks = 2; fake.rank = 0; fake.buf_bytes = ~0ull; fake.f32 = 1;
        aclnnB200SetDecodeGather(&fake);
        uint64_t need = 0;
        aclOpExecutor *probe = nullptr;
        if (local_plan(true, x, weight, scale, offset, out, &need, &probe) == ACLNN_SUCCESS) {
            aclDestroyAclOpExecutor(probe);
            if (need > *ws) *ws = need;
        }
        aclnnB200SetDecodeGather(nullptr);
    }
    *ex = aclnnB200CreateWrapperExecutor(w, free_allreduce);
    if (!*ex) { free_allreduce(w); return ACLNN_ERR_RUNTIME_ERROR; }
    return ACLNN_SUCCESS;
}

aclnnStatus run_chunked(const AllReduceExecutor &w, void *ws, uint64_t wsz, HcclDataType ht, aclrtStream s) {
    OverlapLane *lane = lane_of(w.comm);
    if (!lane) return ACLNN_ERR_RUNTIME_ERROR;
    aclnnStatus st = ACLNN_SUCCESS;
    bool forked = false;
    SmReservation reserve(overlap_sms());
    for (int i = 0; i < w.chunks && st == ACLNN_SUCCESS; ++i) {
        const int64_t r0 = chunk_begin(w.rows, w.chunks, i), r1 = i + 1 == w.chunks ? w.rows : chunk_begin(w.rows, w.chunks, i + 1);
        if (r1 <= r0) continue;
        aclTensor *xs = aclnnB200CreateRowSlice(w.x, r0, r1 - r0), *os = aclnnB200CreateRowSlice(w.out, r0, r1 - r0);
        uint64_t need = 0;
        aclOpExecutor *inner = nullptr;
        st = xs && os ? local_plan(w.weight_only, xs, w.weight, w.scale, w.offset, os, &need, &inner) : ACLNN_ERR_RUNTIME_ERROR;
        if (st == ACLNN_SUCCESS && need > wsz) { aclDestroyAclOpExecutor(inner); st = ACLNN_ERR_PARAM_INVALID; }
        if (st == ACLNN_SUCCESS) st = w.weight_only ? aclnnWeightQuantBatchMatmul(ws, wsz, inner, s) : aclnnQuantMatmul(ws, wsz, inner, s);
        void *data = nullptr;
        int64_t *dims = nullptr;
        uint64_t nd = 0;
        if (st == ACLNN_SUCCESS) st = aclGetRawTensorAddr(w.out, &data);
        if (st == ACLNN_SUCCESS) st = aclGetViewShape(w.out, &dims, &nd);
        if (st == ACLNN_SUCCESS) {
            // the output is contiguous [rows, N] (checked in phase 1 by the local operator): chunk = a byte range
            aclDataType dt = ACL_DT_UNDEFINED;
            aclGetDataType(w.out, &dt);
            const uint64_t esz = dt == ACL_FLOAT ? 4 : 2, n = (uint64_t)dims[1];
            char *chunk = static_cast<char *>(data) + (uint64_t)r0 * n * esz;
            if (aclrtRecordEvent(lane->ready[i], s) != ACL_SUCCESS || aclrtStreamWaitEvent(lane->stream, lane->ready[i]) != ACL_SUCCESS) {
                st = ACLNN_ERR_RUNTIME_ERROR;
            } else {
                forked = true;
                if (HcclAllReduce(chunk, chunk, (uint64_t)(r1 - r0) * n, ht, HCCL_REDUCE_SUM, w.comm, lane->stream) != HCCL_SUCCESS)
                    st = ACLNN_ERR_RUNTIME_ERROR;
            }
        }
        if (xs) aclDestroyTensor(xs);
        if (os) aclDestroyTensor(os);
    }
    // join, also after a failure: a captured stream must not be left forked
    if (forked && (aclrtRecordEvent(lane->done, lane->stream) != ACL_SUCCESS || aclrtStreamWaitEvent(s, lane->done) != ACL_SUCCESS))
        st = st == ACLNN_SUCCESS ? ACLNN_ERR_RUNTIME_ERROR : st;
    return st;
}

aclnnStatus run(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    auto *wp = static_cast<AllReduceExecutor *>(aclnnB200WrapperPayload(e, 1));
    aclDestroyAclOpExecutor(e);   // phase 2 consumes the plan, whatever it was
    if (!wp) return ACLNN_ERR_PARAM_INVALID;
    AllReduceExecutor w = *wp;
    delete wp;
    // read what the all-reduce needs before the local operator runs: the tensors may go away after phase 2
    void *data = nullptr;
    int64_t *dims = nullptr;
    uint64_t nd = 0;
    aclDataType dt = ACL_DT_UNDEFINED;
    aclnnStatus st = aclGetRawTensorAddr(w.out, &data);
    if (st == ACLNN_SUCCESS) st = aclGetViewShape(w.out, &dims, &nd);
    if (st == ACLNN_SUCCESS) st = aclGetDataType(w.out, &dt);
    uint64_t count = 1;
    for (uint64_t i = 0; st == ACLNN_SUCCESS && i < nd; ++i) count *= (uint64_t)dims[i];
    HcclDataType ht = HCCL_DATA_TYPE_FP32;
    if (st == ACLNN_SUCCESS && w.comm && !hccl_type(dt, &ht)) st = ACLNN_ERR_PARAM_INVALID;
    if (st != ACLNN_SUCCESS) {
        aclDestroyAclOpExecutor(w.inner);
        return st;
    }
    if (w.comm && w.chunks > 1 && count > 0) {
        aclDestroyAclOpExecutor(w.inner);   // the whole-problem plan only sized the workspace
        return run_chunked(w, ws, wsz, ht, s);
    }
    // Weight-only decode shapes: the matmul kernel sends its partial rows to the peers' receive windows itself and a
    // receiver kernel sums the ranks' unrounded fp32 partial results (rank order, rounded once) -- one-shot all-reduce over peer
    // memory, no library collective.  Needs the communicator's windows and a plan of the decode kernel that fits the
    // workspace; otherwise the plain sequence below.
    P2pGatherTarget t{};
    if (w.comm && w.weight_only && count > 0 && (dt == ACL_BF16 || dt == ACL_FLOAT16) && hccl_gather_target(w.comm, s, &t) == 1) {
        aclnnB200DecodeGather dg{};
        for (int i = 0; i < 8; ++i) dg.peer[i] = t.peer[i];
        dg.calls = t.calls; dg.nranks = t.nranks; dg.rank = t.rank; dg.buf_bytes = t.buf_bytes; dg.f32 = 1;
        aclnnB200SetDecodeGather(&dg);
        uint64_t need = 0;
        aclOpExecutor *again = nullptr;
        if (local_plan(true, w.x, w.weight, w.scale, w.offset, w.out, &need, &again) == ACLNN_SUCCESS) {
            if (need <= wsz) {
                aclDestroyAclOpExecutor(w.inner);
                w.inner = again;
            } else {
                aclDestroyAclOpExecutor(again);
                aclnnB200SetDecodeGather(nullptr);   // the caller's workspace is too small for that plan: plain sequence
            }
        } else {
            aclnnB200SetDecodeGather(nullptr);
        }
    }
    st = w.weight_only ? aclnnWeightQuantBatchMatmul(ws, wsz, w.inner, s) : aclnnQuantMatmul(ws, wsz, w.inner, s);
    const bool sent = w.weight_only && aclnnB200DecodeGatherConsumed() == 1;
    aclnnB200SetDecodeGather(nullptr);
    if (st == ACLNN_SUCCESS && w.comm && count > 0) {
        if (sent) {
            g_fused_allreduces.fetch_add(1);
            if (hccl_gather_reduce(w.comm, data, count, dt == ACL_BF16 ? 1 : 0, s) != 0) st = ACLNN_ERR_RUNTIME_ERROR;
        } else if (HcclAllReduce(data, data, count, ht, HCCL_REDUCE_SUM, w.comm, s) != HCCL_SUCCESS) {
            st = ACLNN_ERR_RUNTIME_ERROR;
        }
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

// ---- column shards with the gather fused into the matmul's epilogue --------------------------------------
struct GatherExecutor {
    const aclTensor *x = nullptr, *weight = nullptr, *scale = nullptr, *offset = nullptr, *bias = nullptr;
    int64_t group = 0;
    HcclComm comm = nullptr;
    aclTensor *gathered = nullptr;
    uint32_t nranks = 1, rank = 0;
    int64_t rows = 0, cols = 0;        // of one shard
};
void free_gather(void *p) { delete static_cast<GatherExecutor *>(p); }
std::atomic<uint64_t> g_fused_gathers{0};   // calls that took the fused form (diagnostics)

// gathered[rank] as a tensor of its own: [rows, cols] over the same buffer (gathered is contiguous from its data pointer)
aclTensor *own_shard(const GatherExecutor &g) {
    void *data = nullptr;
    aclDataType dt = ACL_DT_UNDEFINED;
    if (aclGetRawTensorAddr(g.gathered, &data) != ACLNN_SUCCESS || !data || aclGetDataType(g.gathered, &dt) != ACLNN_SUCCESS) return nullptr;
    const int64_t dims[2] = {g.rows, g.cols};
    char *base = static_cast<char *>(data) + (size_t)g.rank * g.rows * g.cols * 2;
    return aclCreateTensor(dims, 2, dt, nullptr, 0, ACL_FORMAT_ND, dims, 2, base);
}

aclnnStatus gather_plan(const aclTensor *x, const aclTensor *weight, const aclTensor *scale, const aclTensor *offset, const aclTensor *bias,
                        int64_t group, HcclComm comm, aclTensor *gathered, uint64_t *ws, aclOpExecutor **ex) {
    if (!x || !weight || !scale || !gathered || !ws || !ex) return ACLNN_ERR_PARAM_NULLPTR;
    int64_t *gd = nullptr;
    uint64_t gn = 0;
    aclDataType dt = ACL_DT_UNDEFINED;
    if (aclGetViewShape(gathered, &gd, &gn) != ACLNN_SUCCESS || gn != 3 || aclGetDataType(gathered, &dt) != ACLNN_SUCCESS) return ACLNN_ERR_PARAM_INVALID;
    if (dt != ACL_FLOAT16 && dt != ACL_BF16) return ACLNN_ERR_PARAM_INVALID;
    auto *g = new GatherExecutor();
    g->x = x; g->weight = weight; g->scale = scale; g->offset = offset; g->bias = bias; g->group = group; g->comm = comm; g->gathered = gathered;
    g->rows = gd[1]; g->cols = gd[2];
    if (comm) {
        if (HcclGetRankSize(comm, &g->nranks) != HCCL_SUCCESS || HcclGetRankId(comm, &g->rank) != HCCL_SUCCESS) { delete g; return ACLNN_ERR_RUNTIME_ERROR; }
    }
    if ((int64_t)g->nranks != gd[0]) { delete g; return ACLNN_ERR_PARAM_INVALID; }
    // the local plan, with and without the gathering epilogue: the workspace must serve both (which one phase 2 takes
    // depends on whether the windows can be set up, known only there)
    aclTensor *out = own_shard(*g);
    if (!out) { delete g; return ACLNN_ERR_PARAM_INVALID; }
    uint64_t need_plain = 0, need_gather = 0;
    aclOpExecutor *probe = nullptr;
    aclnnStatus st = aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(x, weight, scale, offset, bias, group, out, &need_plain, &probe);
    if (st == ACLNN_SUCCESS) {
        aclDestroyAclOpExecutor(probe);
        aclnnB200DecodeGather fake{};
        fake.nranks = g->nranks > 1 ? g->nranks : 2; fake.rank = 0; fake.buf_bytes = ~0ull;
        aclnnB200SetDecodeGather(&fake);
        st = aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(x, weight, scale, offset, bias, group, out, &need_gather, &probe);
        aclnnB200SetDecodeGather(nullptr);
        if (st == ACLNN_SUCCESS) aclDestroyAclOpExecutor(probe);
    }
    aclDestroyTensor(out);
    if (st != ACLNN_SUCCESS) { delete g; return st; }
    *ws = need_plain > need_gather ? need_plain : need_gather;
    *ex = aclnnB200CreateWrapperExecutor(g, free_gather);
    if (!*ex) { delete g; return ACLNN_ERR_RUNTIME_ERROR; }
    return ACLNN_SUCCESS;
}

aclnnStatus gather_run(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) {
    if (!e) return ACLNN_ERR_PARAM_NULLPTR;
    auto *gp = static_cast<GatherExecutor *>(aclnnB200WrapperPayload(e, 1));
    aclDestroyAclOpExecutor(e);
    if (!gp) return ACLNN_ERR_PARAM_INVALID;
    const GatherExecutor g = *gp;
    delete gp;
    aclTensor *out = own_shard(g);
    if (!out) return ACLNN_ERR_PARAM_INVALID;
    void *gathered_data = nullptr;
    aclGetRawTensorAddr(g.gathered, &gathered_data);
    // the fused form, if this communicator has its windows
    P2pGatherTarget t{};
    const bool windows = g.comm && g.nranks > 1 && hccl_gather_target(g.comm, s, &t) == 1;
    if (windows) {
        aclnnB200DecodeGather dg{};
        for (int i = 0; i < 8; ++i) dg.peer[i] = t.peer[i];
        dg.calls = t.calls; dg.nranks = t.nranks; dg.rank = t.rank; dg.buf_bytes = t.buf_bytes;
        aclnnB200SetDecodeGather(&dg);
    }
    uint64_t need = 0;
    aclOpExecutor *inner = nullptr;
    aclnnStatus st = aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(g.x, g.weight, g.scale, g.offset, g.bias, g.group, out, &need, &inner);
    if (st == ACLNN_SUCCESS && need > wsz) { aclDestroyAclOpExecutor(inner); st = ACLNN_ERR_PARAM_INVALID; }
    if (st == ACLNN_SUCCESS) st = aclnnWeightQuantBatchMatmulV2Ex(ws, wsz, inner, s);
    const bool fused = windows && aclnnB200DecodeGatherConsumed() == 1;
    if (windows) aclnnB200SetDecodeGather(nullptr);
    aclDestroyTensor(out);
    if (st != ACLNN_SUCCESS || !g.comm || g.nranks < 2) return st;
    const uint64_t per_rank = (uint64_t)g.rows * (uint64_t)g.cols;
    if (fused) {
        g_fused_gathers.fetch_add(1);
        return hccl_gather_unpack(g.comm, gathered_data, per_rank, s) == 0 ? ACLNN_SUCCESS : ACLNN_ERR_RUNTIME_ERROR;
    }
    // the plain sequence: the local shard is in place already, the library gathers in place
    aclDataType dt = ACL_DT_UNDEFINED;
    aclGetDataType(g.gathered, &dt);
    char *mine = static_cast<char *>(gathered_data) + (size_t)g.rank * per_rank * 2;
    return HcclAllGather(mine, gathered_data, per_rank, dt == ACL_BF16 ? HCCL_DATA_TYPE_BFP16 : HCCL_DATA_TYPE_FP16, g.comm, s) == HCCL_SUCCESS
               ? ACLNN_SUCCESS : ACLNN_ERR_RUNTIME_ERROR;
}

}  // namespace

extern "C" {

aclnnStatus aclnnB200WeightQuantMatmulAllGatherGetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *antiquantScale,
        const aclTensor *antiquantOffsetOptional, const aclTensor *biasOptional, int64_t antiquantGroupSize, HcclComm comm,
        aclTensor *gathered, uint64_t *ws, aclOpExecutor **ex) {
    return gather_plan(x, weight, antiquantScale, antiquantOffsetOptional, biasOptional, antiquantGroupSize, comm, gathered, ws, ex);
}
aclnnStatus aclnnB200WeightQuantMatmulAllGather(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return gather_run(ws, wsz, e, s); }
uint64_t aclnnB200FusedGatherCount(void) { return g_fused_gathers.load(); }
uint64_t aclnnB200FusedAllReduceCount(void) { return g_fused_allreduces.load(); }

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
        return wrap(st, inner, comm, x, weight, scale, nullptr, out, false, ws, ex);                                 \
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
    return wrap(st, inner, comm, x, weight, antiquantScale, antiquantOffset, out, true, ws, ex);
}
aclnnStatus aclnnWeightQuantMatmulAllReduce(void *ws, uint64_t wsz, aclOpExecutor *e, aclrtStream s) { return run(ws, wsz, e, s); }

}  // extern "C"
