/* A plain C client of the AscendCL ABI, the way an Ascend-API program drives the weight-only
 * quantized matmul with host data (the reference's test harness does the same steps,
 * tests/harness.h:62-70): copy the activations to the device, phase 1 (workspace size + executor),
 * phase 2 (enqueue), copy the result back.  It touches the library only through its exported C
 * symbols; the benchmark's end-to-end leg calls it so that the timed region holds what a compiled
 * client pays, not the overhead of a Python loop.
 *
 * The pass is software-pipelined over three streams the way a serving loop does it: the copy-in of
 * call i+1 and the copy-out of call i-1 run beside the matmul of call i (two activation buffers,
 * two output buffers, events between the streams).  Every call still pays its own host-to-device
 * copy, both phases of the operator and its device-to-host copy, and the pass ends with everything
 * synchronised.  The pass can also be captured once into a model and replayed, which removes the
 * per-call host work and the gaps between dependent launches on different streams. */
#include <stddef.h>
#include <stdint.h>

#include "acl/acl.h"
#include "aclnnop/aclnn_quant_matmul.h"

#define QMM_CLIENT_API __attribute__((visibility("default")))

static aclrtStream g_in, g_out;          /* copy streams, created on first use */
static aclrtEvent g_ev_in[2], g_ev_comp[2], g_ev_out[2], g_ev_fork, g_ev_join;
static int g_ready;

static int client_setup(void) {
    if (g_ready) return 0;
    if (aclrtCreateStream(&g_in) != ACL_SUCCESS || aclrtCreateStream(&g_out) != ACL_SUCCESS) return 1;
    for (int b = 0; b < 2; ++b) {
        if (aclrtCreateEvent(&g_ev_in[b]) != ACL_SUCCESS || aclrtCreateEvent(&g_ev_comp[b]) != ACL_SUCCESS ||
            aclrtCreateEvent(&g_ev_out[b]) != ACL_SUCCESS) return 1;
    }
    if (aclrtCreateEvent(&g_ev_fork) != ACL_SUCCESS || aclrtCreateEvent(&g_ev_join) != ACL_SUCCESS) return 1;
    g_ready = 1;
    return 0;
}

/* Enqueues one pass over n argument sets (no synchronisation).  With `forked` set the copy-in stream
 * first waits for an event recorded on `stream` and both copy streams are joined back into `stream`
 * at the end, which is what stream capture needs (every captured stream must fork from and rejoin the
 * capturing one). */
static int enqueue_pass(int n, const void *const *host_x, size_t x_bytes, void *const *dev_x, const aclTensor *const *x,
                        const aclTensor *const *weight, const aclTensor *const *scale, const aclTensor *const *offset,
                        const aclTensor *const *bias, int64_t group, aclTensor *const *out, const void *const *dev_out,
                        void *host_out, size_t out_bytes, void *workspace, uint64_t workspace_bytes, aclrtStream stream,
                        int forked) {
    aclError e;
    if (forked) {
        if ((e = aclrtRecordEvent(g_ev_fork, stream)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtStreamWaitEvent(g_in, g_ev_fork)) != ACL_SUCCESS) return (int)e;
    }
    for (int i = 0; i < n; ++i) {
        const int b = i & 1;
        /* copy-in stream: the buffer is free once call i-2 has run */
        if (i >= 2 && (e = aclrtStreamWaitEvent(g_in, g_ev_comp[b])) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtMemcpyAsync(dev_x[b], x_bytes, host_x[i], x_bytes, ACL_MEMCPY_HOST_TO_DEVICE, g_in)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtRecordEvent(g_ev_in[b], g_in)) != ACL_SUCCESS) return (int)e;
        /* compute stream: needs the activations, and the output buffer drained by call i-2's copy-out */
        if ((e = aclrtStreamWaitEvent(stream, g_ev_in[b])) != ACL_SUCCESS) return (int)e;
        if (i >= 2 && (e = aclrtStreamWaitEvent(stream, g_ev_out[b])) != ACL_SUCCESS) return (int)e;
        uint64_t need = 0;
        aclOpExecutor *ex = NULL;
        aclnnStatus st = aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(x[b], weight[i], scale[i], offset ? offset[i] : NULL,
                                                                         bias ? bias[i] : NULL, group, out[b], &need, &ex);
        if (st != 0) return (int)st;
        if (need > workspace_bytes) { aclDestroyAclOpExecutor(ex); return 161002; }
        st = aclnnWeightQuantBatchMatmulV2Ex(workspace, workspace_bytes, ex, stream);
        if (st != 0) return (int)st;
        if ((e = aclrtRecordEvent(g_ev_comp[b], stream)) != ACL_SUCCESS) return (int)e;
        /* copy-out stream */
        if ((e = aclrtStreamWaitEvent(g_out, g_ev_comp[b])) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtMemcpyAsync(host_out, out_bytes, dev_out[b], out_bytes, ACL_MEMCPY_DEVICE_TO_HOST, g_out)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtRecordEvent(g_ev_out[b], g_out)) != ACL_SUCCESS) return (int)e;
    }
    if (forked) {
        if ((e = aclrtRecordEvent(g_ev_join, g_in)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtStreamWaitEvent(stream, g_ev_join)) != ACL_SUCCESS) return (int)e;
        if (n > 0 && (e = aclrtStreamWaitEvent(stream, g_ev_out[(n - 1) & 1])) != ACL_SUCCESS) return (int)e;
        if (n > 1 && (e = aclrtStreamWaitEvent(stream, g_ev_out[n & 1])) != ACL_SUCCESS) return (int)e;
    }
    return 0;
}

/* One pass over n argument sets.  dev_x[b] / x[b] and dev_out[b] / out[b] (b = 0, 1) are the two
 * activation and output buffers with their tensors; call i uses buffer i % 2.  host_x[i] is copied
 * in before call i, the output is copied to host_out after it.  Returns 0, or the first status
 * that was not success.  The workspace must hold workspace_bytes; a call that asks for more returns
 * 161002 from here.  Not re-entrant (one set of streams and events per process). */
QMM_CLIENT_API int qmmClientWeightQuantPass(int n, const void *const *host_x, size_t x_bytes, void *const *dev_x,
                                            const aclTensor *const *x, const aclTensor *const *weight,
                                            const aclTensor *const *scale, const aclTensor *const *offset,
                                            const aclTensor *const *bias, int64_t group, aclTensor *const *out,
                                            const void *const *dev_out, void *host_out, size_t out_bytes, void *workspace,
                                            uint64_t workspace_bytes, aclrtStream stream) {
    if (client_setup()) return 361001;
    const int st = enqueue_pass(n, host_x, x_bytes, dev_x, x, weight, scale, offset, bias, group, out, dev_out, host_out, out_bytes,
                                workspace, workspace_bytes, stream, 0);
    if (st != 0) return st;
    aclError e = aclrtSynchronizeStream(g_out);
    if (e == ACL_SUCCESS) e = aclrtSynchronizeStream(stream);
    if (e == ACL_SUCCESS) e = aclrtSynchronizeStream(g_in);
    return (int)e;
}

/* The same pass captured once into a model (aclmdlRICaptureBegin / End, the way the reference's
 * tests/test_graph.cpp captures a decode step): phase 1 of every call runs here, on the host, at
 * capture time; a replay re-issues the copies from the same host buffers, the kernels and the copies
 * back.  Run the pass directly once before capturing (first launches set kernel attributes).  The
 * host buffers, device buffers, tensors' data and the workspace must stay valid while the model is
 * used.  On failure the capture is ended and its model dropped. */
QMM_CLIENT_API int qmmClientWeightQuantCapture(int n, const void *const *host_x, size_t x_bytes, void *const *dev_x,
                                               const aclTensor *const *x, const aclTensor *const *weight,
                                               const aclTensor *const *scale, const aclTensor *const *offset,
                                               const aclTensor *const *bias, int64_t group, aclTensor *const *out,
                                               const void *const *dev_out, void *host_out, size_t out_bytes, void *workspace,
                                               uint64_t workspace_bytes, aclrtStream stream, aclmdlRI *model) {
    if (!model) return 161001;
    *model = NULL;
    if (client_setup()) return 361001;
    aclError e = aclmdlRICaptureBegin(stream, ACL_MODEL_RI_CAPTURE_MODE_RELAXED);
    if (e != ACL_SUCCESS) return (int)e;
    const int st = enqueue_pass(n, host_x, x_bytes, dev_x, x, weight, scale, offset, bias, group, out, dev_out, host_out, out_bytes,
                                workspace, workspace_bytes, stream, 1);
    e = aclmdlRICaptureEnd(stream, model);
    if (st != 0) {
        if (e == ACL_SUCCESS) aclmdlRIDestroy(*model);
        *model = NULL;
        return st;
    }
    return (int)e;
}

/* ---- a whole decode step of n calls -----------------------------------------------------------------
 * The same per-call work (copy in, phase 1, phase 2, copy out) arranged the way a serving loop arranges a
 * step of many layers: every call has its own activation and output buffer (no reuse inside the step), the
 * host buffers of the step are one contiguous block each, and the copies are issued in groups of `per_group`
 * calls -- the copy-in of a group is one transfer on the copy-in stream, the matmuls of the group follow on
 * `stream` back to back (nothing between them, so each one's start-up overlaps its predecessor's end), the
 * copy-out of the group is one transfer on the copy-out stream.  Group k+1's copy-in and group k-1's
 * copy-out run beside group k's matmuls.  Every byte of every call still crosses the bus inside the step. */
#define QMM_MAX_GROUPS 64
static aclrtEvent g_ev_gin[QMM_MAX_GROUPS], g_ev_gcomp[QMM_MAX_GROUPS];
static int g_groups_ready;

static int step_setup(void) {
    if (client_setup()) return 1;
    if (g_groups_ready) return 0;
    for (int k = 0; k < QMM_MAX_GROUPS; ++k)
        if (aclrtCreateEvent(&g_ev_gin[k]) != ACL_SUCCESS || aclrtCreateEvent(&g_ev_gcomp[k]) != ACL_SUCCESS) return 1;
    g_groups_ready = 1;
    return 0;
}

static int enqueue_step(int n, int per_group, const void *host_x, size_t x_bytes, void *dev_x, const aclTensor *const *x,
                        const aclTensor *const *weight, const aclTensor *const *scale, const aclTensor *const *offset,
                        const aclTensor *const *bias, int64_t group, aclTensor *const *out, const void *dev_out, void *host_out,
                        size_t out_bytes, void *workspace, uint64_t workspace_bytes, aclrtStream stream, int forked) {
    aclError e;
    if (n < 1 || per_group < 1 || (n + per_group - 1) / per_group > QMM_MAX_GROUPS) return 161002;
    const int groups = (n + per_group - 1) / per_group;
    if (forked) {
        if ((e = aclrtRecordEvent(g_ev_fork, stream)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtStreamWaitEvent(g_in, g_ev_fork)) != ACL_SUCCESS) return (int)e;
    }
    /* all copies in, group by group, as early as the bus allows */
    for (int k = 0; k < groups; ++k) {
        const int first = k * per_group, cnt = (first + per_group <= n ? per_group : n - first);
        if ((e = aclrtMemcpyAsync((char *)dev_x + (size_t)first * x_bytes, cnt * x_bytes, (const char *)host_x + (size_t)first * x_bytes,
                                  cnt * x_bytes, ACL_MEMCPY_HOST_TO_DEVICE, g_in)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtRecordEvent(g_ev_gin[k], g_in)) != ACL_SUCCESS) return (int)e;
    }
    for (int k = 0; k < groups; ++k) {
        const int first = k * per_group, cnt = (first + per_group <= n ? per_group : n - first);
        if ((e = aclrtStreamWaitEvent(stream, g_ev_gin[k])) != ACL_SUCCESS) return (int)e;
        for (int i = first; i < first + cnt; ++i) {
            uint64_t need = 0;
            aclOpExecutor *ex = NULL;
            aclnnStatus st = aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(x[i], weight[i], scale[i], offset ? offset[i] : NULL,
                                                                             bias ? bias[i] : NULL, group, out[i], &need, &ex);
            if (st != 0) return (int)st;
            if (need > workspace_bytes) { aclDestroyAclOpExecutor(ex); return 161002; }
            st = aclnnWeightQuantBatchMatmulV2Ex(workspace, workspace_bytes, ex, stream);
            if (st != 0) return (int)st;
        }
        if ((e = aclrtRecordEvent(g_ev_gcomp[k], stream)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtStreamWaitEvent(g_out, g_ev_gcomp[k])) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtMemcpyAsync((char *)host_out + (size_t)first * out_bytes, cnt * out_bytes,
                                  (const char *)dev_out + (size_t)first * out_bytes, cnt * out_bytes, ACL_MEMCPY_DEVICE_TO_HOST,
                                  g_out)) != ACL_SUCCESS) return (int)e;
    }
    if (forked) {
        if ((e = aclrtRecordEvent(g_ev_join, g_in)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtStreamWaitEvent(stream, g_ev_join)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtRecordEvent(g_ev_out[0], g_out)) != ACL_SUCCESS) return (int)e;
        if ((e = aclrtStreamWaitEvent(stream, g_ev_out[0])) != ACL_SUCCESS) return (int)e;
    }
    return 0;
}

/* One step of n calls, enqueued and waited for.  host_x / dev_x are [n][x_bytes], dev_out / host_out [n][out_bytes];
 * x[i] and out[i] are the tensors over call i's slices, weight[i] / scale[i] its weights.  The calls of one step share
 * `workspace` (they run in order on `stream`).  Returns 0 or the first status that was not success. */
QMM_CLIENT_API int qmmClientWeightQuantStep(int n, int per_group, const void *host_x, size_t x_bytes, void *dev_x,
                                            const aclTensor *const *x, const aclTensor *const *weight, const aclTensor *const *scale,
                                            const aclTensor *const *offset, const aclTensor *const *bias, int64_t group,
                                            aclTensor *const *out, const void *dev_out, void *host_out, size_t out_bytes,
                                            void *workspace, uint64_t workspace_bytes, aclrtStream stream) {
    if (step_setup()) return 361001;
    const int st = enqueue_step(n, per_group, host_x, x_bytes, dev_x, x, weight, scale, offset, bias, group, out, dev_out, host_out,
                                out_bytes, workspace, workspace_bytes, stream, 0);
    if (st != 0) return st;
    aclError e = aclrtSynchronizeStream(g_out);
    if (e == ACL_SUCCESS) e = aclrtSynchronizeStream(stream);
    if (e == ACL_SUCCESS) e = aclrtSynchronizeStream(g_in);
    return (int)e;
}

/* The same step captured once into a model (see qmmClientWeightQuantCapture); replay with qmmClientReplay. */
QMM_CLIENT_API int qmmClientWeightQuantStepCapture(int n, int per_group, const void *host_x, size_t x_bytes, void *dev_x,
                                                   const aclTensor *const *x, const aclTensor *const *weight,
                                                   const aclTensor *const *scale, const aclTensor *const *offset,
                                                   const aclTensor *const *bias, int64_t group, aclTensor *const *out,
                                                   const void *dev_out, void *host_out, size_t out_bytes, void *workspace,
                                                   uint64_t workspace_bytes, aclrtStream stream, aclmdlRI *model) {
    if (!model) return 161001;
    *model = NULL;
    if (step_setup()) return 361001;
    aclError e = aclmdlRICaptureBegin(stream, ACL_MODEL_RI_CAPTURE_MODE_RELAXED);
    if (e != ACL_SUCCESS) return (int)e;
    const int st = enqueue_step(n, per_group, host_x, x_bytes, dev_x, x, weight, scale, offset, bias, group, out, dev_out, host_out,
                                out_bytes, workspace, workspace_bytes, stream, 1);
    e = aclmdlRICaptureEnd(stream, model);
    if (st != 0) {
        if (e == ACL_SUCCESS) aclmdlRIDestroy(*model);
        *model = NULL;
        return st;
    }
    return (int)e;
}

/* Replays a captured pass on `stream` and waits for it. */
QMM_CLIENT_API int qmmClientReplay(aclmdlRI model, aclrtStream stream) {
    aclError e = aclmdlRIExecuteAsync(model, stream);
    if (e == ACL_SUCCESS) e = aclrtSynchronizeStream(stream);
    return (int)e;
}
