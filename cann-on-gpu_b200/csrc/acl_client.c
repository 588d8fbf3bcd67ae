/* A plain C client of the AscendCL ABI, the way an Ascend-API program drives the weight-only
 * quantized matmul with host data (the reference's test harness does the same steps,
 * tests/harness.h:62-70): copy the activations to the device, phase 1 (workspace size + executor),
 * phase 2 (enqueue), copy the result back, and synchronise the stream once per pass.  It touches
 * the library only through its exported C symbols; the benchmark's end-to-end leg calls it so that
 * the timed region holds what a compiled client pays, not the overhead of a Python loop. */
#include <stddef.h>
#include <stdint.h>

#include "acl/acl.h"
#include "aclnnop/aclnn_quant_matmul.h"

#define QMM_CLIENT_API __attribute__((visibility("default")))

/* One pass over n argument sets that share the activation buffer dev_x / tensor x and the output
 * tensor out.  host_x[i] is copied to dev_x before call i, the output is copied to host_out after
 * it.  Returns 0, or the first status that was not success.  The workspace must hold
 * workspace_bytes; a call that asks for more returns 161002 from here. */
QMM_CLIENT_API int qmmClientWeightQuantPass(int n, const void *const *host_x, size_t x_bytes, void *dev_x, const aclTensor *x,
                                            const aclTensor *const *weight, const aclTensor *const *scale,
                                            const aclTensor *const *offset, const aclTensor *const *bias, int64_t group,
                                            aclTensor *out, const void *dev_out, void *host_out, size_t out_bytes,
                                            void *workspace, uint64_t workspace_bytes, aclrtStream stream) {
    for (int i = 0; i < n; ++i) {
        aclError e = aclrtMemcpyAsync(dev_x, x_bytes, host_x[i], x_bytes, ACL_MEMCPY_HOST_TO_DEVICE, stream);
        if (e != ACL_SUCCESS) return (int)e;
        uint64_t need = 0;
        aclOpExecutor *ex = NULL;
        aclnnStatus st = aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(x, weight[i], scale[i], offset ? offset[i] : NULL,
                                                                         bias ? bias[i] : NULL, group, out, &need, &ex);
        if (st != 0) return (int)st;
        if (need > workspace_bytes) return 161002;
        st = aclnnWeightQuantBatchMatmulV2Ex(workspace, workspace_bytes, ex, stream);
        if (st != 0) return (int)st;
        e = aclrtMemcpyAsync(host_out, out_bytes, dev_out, out_bytes, ACL_MEMCPY_DEVICE_TO_HOST, stream);
        if (e != ACL_SUCCESS) return (int)e;
    }
    return (int)aclrtSynchronizeStream(stream);
}
