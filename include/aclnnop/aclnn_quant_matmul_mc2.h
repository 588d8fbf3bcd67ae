/*
 * aclnnop/aclnn_quant_matmul_mc2.h -- quantized matmuls followed by an all-reduce over the ranks of a
 * communicator (K-split tensor parallelism: every rank multiplies its slice of K, the partial
 * outputs are summed).  Exported by libhccl.so, which runs the local operator of libascendcl.so and
 * then HcclAllReduce (NCCL over NVLink) on the caller's stream.  comm == NULL: local result only.
 * Same names and argument order as the reference's include/aclnnop/aclnn_mc2.h:22-24,88-91
 * (cuda/src/ops/mc2_ext.cu:67-87,185-195; cuda/src/ops/matmul.cu:1304-1319).
 * Column sharding with no collective, not this, is the scaling path of the library.
 */
#ifndef B200_ACLNN_QUANT_MATMUL_MC2_H
#define B200_ACLNN_QUANT_MATMUL_MC2_H

#include "aclnnop/aclnn_quant_matmul.h"
#include "hccl/hccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ACLNN_QMM_ALLREDUCE(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, \
        const aclTensor *scale, HcclComm comm, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor); \
    ACL_FUNC_VISIBILITY aclnnStatus NAME(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream);
B200_ACLNN_QMM_ALLREDUCE(aclnnQuantMatmulAllReduce)
B200_ACLNN_QMM_ALLREDUCE(aclnnQuantMatmulAllReduceV2)
B200_ACLNN_QMM_ALLREDUCE(aclnnQuantMatmulAllReduceV3)
B200_ACLNN_QMM_ALLREDUCE(aclnnQuantMatmulAllReduceV4)

ACL_FUNC_VISIBILITY aclnnStatus aclnnWeightQuantMatmulAllReduceGetWorkspaceSize(const aclTensor *x, const aclTensor *weight,
    const aclTensor *antiquantScale, const aclTensor *antiquantOffset, HcclComm comm, aclTensor *out,
    uint64_t *workspaceSize, aclOpExecutor **executor);
ACL_FUNC_VISIBILITY aclnnStatus aclnnWeightQuantMatmulAllReduce(void *workspace, uint64_t workspaceSize,
    aclOpExecutor *executor, aclrtStream stream);

/* W8A8 matmul -> all-reduce (sum over the ranks of comm; none when comm == NULL) -> residual add + RMS
 * norm: y = rmsnorm(allreduce(x @ weight * scale) + residual) * gamma, residualSum = the sum before the
 * norm.  y, residual, residualSum [M,N] of one 16/32-bit float type; gamma [N] or NULL.  The partial
 * output is kept in the workspace (phase 1 reports its size).  The reference's Inplace form (y over the
 * int8 x) has no consistent types and is not exported.
 * Same names and argument order as the reference's cuda/src/ops/matmul.cu:1344-1370 (its
 * composition: matmul.cu:1222-1233). */
ACL_FUNC_VISIBILITY aclnnStatus aclnnQuantMatmulAllReduceAddRmsNormGetWorkspaceSize(const aclTensor *x, const aclTensor *weight,
    const aclTensor *scale, const aclTensor *residual, const aclTensor *gamma, double eps, HcclComm comm, aclTensor *y,
    aclTensor *residualSum, uint64_t *workspaceSize, aclOpExecutor **executor);
ACL_FUNC_VISIBILITY aclnnStatus aclnnQuantMatmulAllReduceAddRmsNorm(void *workspace, uint64_t workspaceSize,
    aclOpExecutor *executor, aclrtStream stream);
/* Column-partitioned weight-only matmul with the gather of the output shards fused into its epilogue (no counterpart in
 * the reference, which offers only the K split above; HcclAllGather, cuda/src/hccl.cu:108-113, is the unfused form).
 * Rank r of comm holds columns [r N/g, (r+1) N/g) of the layer: weight [K, N/g], scale / offset / bias for those columns;
 * x [M,K] is the same on every rank.  gathered is [g][M][N/g] (rank-major, contiguous, the activation type): rank r's own
 * shard is written into gathered[r] by its matmul, and the other ranks' shards arrive through receive windows in peer
 * memory -- the decode kernel stores every finished row straight into the peers' windows, and a small receiver kernel
 * behind it copies them into gathered (csrc/hccl_p2p.cu).  Up to 16 rows, 16-bit activations, g <= 8 and
 * g M N/g <= 2 Mi elements take that form; anything else (and comm windows that cannot be set up) runs the local matmul
 * followed by HcclAllGather, with the same result.  The first call on a communicator sets the windows up collectively:
 * make it outside stream capture.  Every rank must make the same calls in the same order. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnB200WeightQuantMatmulAllGatherGetWorkspaceSize(const aclTensor *x, const aclTensor *weight,
    const aclTensor *antiquantScale, const aclTensor *antiquantOffsetOptional, const aclTensor *biasOptional,
    int64_t antiquantGroupSize, HcclComm comm, aclTensor *gathered, uint64_t *workspaceSize, aclOpExecutor **executor);
ACL_FUNC_VISIBILITY aclnnStatus aclnnB200WeightQuantMatmulAllGather(void *workspace, uint64_t workspaceSize,
    aclOpExecutor *executor, aclrtStream stream);
/* Diagnostics: how many of this process's aclnnB200WeightQuantMatmulAllGather calls took the fused form so far. */
ACL_FUNC_VISIBILITY uint64_t aclnnB200FusedGatherCount(void);
/* aclnnWeightQuantMatmulAllReduce on decode shapes (up to 16 rows, 16-bit types) takes a fused form too: the decode
 * kernel sends its partial rows, unrounded fp32, to the receive windows and a receiver kernel sums the ranks' partial
 * results in rank order and rounds once (a one-shot all-reduce over peer memory instead of HcclAllReduce of 16-bit
 * partial outputs, which rounds every partial result first).  Diagnostics: how
 * many calls of this process took that form. */
ACL_FUNC_VISIBILITY uint64_t aclnnB200FusedAllReduceCount(void);
#ifdef __cplusplus
}
#endif
#endif
