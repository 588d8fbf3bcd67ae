/*
 * hccl/hccl.h -- collective entry points used to gather column-sharded matmul outputs.
 * Same names and argument order as the reference's include/hccl/hccl.h:17-43; implemented over
 * NCCL (reference: cuda/src/hccl.cu:47-172).
 */
#ifndef B200_HCCL_H
#define B200_HCCL_H

#include "hccl/hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *aclrtStreamH; /* = aclrtStream */

/* reference: cuda/src/hccl.cu:47-60 (root info carries the NCCL unique id). */
HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo);
HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm);
HcclResult HcclCommDestroy(HcclComm comm);
/* reference: cuda/src/hccl.cu:101-120. */
HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType,
                         HcclReduceOp op, HcclComm comm, aclrtStreamH stream);
HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType,
                         HcclComm comm, aclrtStreamH stream);
HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                             HcclReduceOp op, HcclComm comm, aclrtStreamH stream);
HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root,
                         HcclComm comm, aclrtStreamH stream);
/* No counterpart in the reference.  The gathering matmul (aclnnB200WeightQuantMatmulAllGather,
 * aclnnop/aclnn_quant_matmul_mc2.h) receives the other ranks' output shards through windows in peer memory; a poll for a
 * peer's data inside its receiver kernel gives up after about a second and leaves 0x500 + the peer's rank here; 0 = none. */
uint32_t HcclB200P2pStatus(void);
/* Test hook: runs the receiver kernel on a window whose peer never sends, with a poll limit of waitNs nanoseconds, and
 * returns the code it left (0x501) -- the failure path of the fused gather, exercised on one GPU without a fault. */
uint32_t HcclB200TestReceiverTimeout(uint64_t waitNs);
/* reference: cuda/src/hccl.cu:164-172. */
HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize);
HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank);

#ifdef __cplusplus
}
#endif
#endif
