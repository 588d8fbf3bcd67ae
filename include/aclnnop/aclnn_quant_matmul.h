/*
 * aclnn_quant_matmul.h -- the quantized-matmul family of the aclnn two-phase operator ABI,
 * implemented with hand-written sm_100a kernels.
 *
 * Every operator is a pair
 *     aclnnStatus aclnnXxxGetWorkspaceSize(<tensors...>, uint64_t *workspaceSize, aclOpExecutor **executor);
 *     aclnnStatus aclnnXxx(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream);
 * Phase 1 runs on the host only, validates, and returns the scratch bytes the caller must provide.
 * Phase 2 enqueues kernels on `stream` (a cudaStream_t), never synchronises or allocates, and
 * consumes the executor (one executor = one launch).  Status codes: 0 ok, 161001 null pointer,
 * 161002 invalid parameter, 361001 runtime error.
 *
 * Each declaration cites the reference interface it replaces (paths inside Cryspia/cann-on-gpu).
 */
#ifndef B200_ACLNN_QUANT_MATMUL_H
#define B200_ACLNN_QUANT_MATMUL_H

#include "aclnn/acl_meta.h"

/* aclnn status codes (same values as the reference's cuda/src/internal.h:16-19). */
#ifndef ACLNN_SUCCESS
#define ACLNN_SUCCESS 0
#define ACLNN_ERR_PARAM_NULLPTR 161001
#define ACLNN_ERR_PARAM_INVALID 161002
#define ACLNN_ERR_RUNTIME_ERROR 361001
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ACLNN_RUN(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream);

/* ---- Weight-only quantized matmul (W8A16 / W4A16) ---------------------------------------------
 * out[M,N] = x[M,K] @ ((weight[K,N] - antiquantOffset) * antiquantScale)
 * weight: ACL_INT8, or ACL_INT4 packed two per byte (linear index k*N+n; even index = low nibble,
 * two's complement).  antiquantScale / antiquantOffset: [N] (per channel) or [K/g, N] (group-wise,
 * g = K / rows).  x/out/scale/offset: ACL_FLOAT16, ACL_BF16 or ACL_FLOAT (all the same type).
 * Replaces include/aclnnop/aclnn_ops.h:1041-1043 and the V2/V3 aliases at :1052-1062
 * (implementation cuda/src/ops/matmul.cu:758-796, cuda/src/ops/quant.cu:216-223);
 * ...Nz replaces cuda/src/ops/matmul.cu:1450-1454. */
#define B200_ACLNN_WQBMM(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, \
        const aclTensor *antiquantScale, const aclTensor *antiquantOffset, aclTensor *out, \
        uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_WQBMM(aclnnWeightQuantBatchMatmul)
B200_ACLNN_WQBMM(aclnnWeightQuantBatchMatmulV2)
B200_ACLNN_WQBMM(aclnnWeightQuantBatchMatmulV3)
B200_ACLNN_WQBMM(aclnnWeightQuantBatchMatmulNz)

/* Extended form: adds the optional bias [N] (same type as x) and an explicit group size
 * (0 = infer from antiquantScale's shape).  The reference ABI has no slot for these
 * (cuda/src/ops/matmul.cu:761-767 rejects them); the old names forward here with nulls. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(const aclTensor *x, const aclTensor *weight,
    const aclTensor *antiquantScale, const aclTensor *antiquantOffsetOptional, const aclTensor *biasOptional,
    int64_t antiquantGroupSize, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnWeightQuantBatchMatmulV2Ex)

/* ---- W8A8 quantized matmul ----------------------------------------------------------------------
 * acc[M,N] = int32( x[M,K] int8 @ weight[K,N] int8 )            (exact)
 * out      = T( float(acc) * scale[n] )                          (reference epilogue, matmul.cu:327-330)
 * scale: [N], ACL_FLOAT16 / ACL_BF16 / ACL_FLOAT.  out: ACL_FLOAT16 / ACL_BF16 / ACL_FLOAT.
 * Replaces include/aclnnop/aclnn_ops.h:1044-1060 (cuda/src/ops/matmul.cu:799-859 and the aliases at
 * cuda/src/ops/quant.cu:204-213,226-230; WeightNz cuda/src/ops/matmul.cu:1457-1461; Fused* and
 * MatmulCompressDequant cuda/src/ops/matmul.cu:1156-1161; Sparse4to2* / DualLevel*
 * include/aclnnop/aclnn_mc2.h:92-95). */
#define B200_ACLNN_QMM(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, \
        const aclTensor *scale, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_QMM(aclnnQuantMatmul)
B200_ACLNN_QMM(aclnnQuantMatmulV2)
B200_ACLNN_QMM(aclnnQuantMatmulV3)
B200_ACLNN_QMM(aclnnQuantMatmulV4)
B200_ACLNN_QMM(aclnnQuantMatmulV5)
B200_ACLNN_QMM(aclnnQuantMatmulDequant)
B200_ACLNN_QMM(aclnnQuantMatmulWeightNz)
B200_ACLNN_QMM(aclnnFusedQuantMatmul)
B200_ACLNN_QMM(aclnnFusedQuantMatmulWeightNz)
B200_ACLNN_QMM(aclnnMatmulCompressDequant)
B200_ACLNN_QMM(aclnnSparse4to2QuantMatmulWeightNz)
B200_ACLNN_QMM(aclnnDualLevelQuantMatmulWeightNz)
/* out += dequant(x @ weight, scale)  -- replaces aclnn_ops.h:1067-1069 (cuda/src/ops/quant.cu:273-299). */
B200_ACLNN_QMM(aclnnQuantBatchMatmulInplaceAdd)
/* weight given as [N,K]  -- replaces cuda/src/ops/quant.cu:303-326. */
B200_ACLNN_QMM(aclnnTransposeQuantBatchMatMul)
/* batched int8: self[B,M,K] @ other[B,K,N] * scale[N]  -- replaces aclnn_ops.h:1997-1998
 * (cuda/src/ops/matmul.cu:1097-1149). */
B200_ACLNN_QMM(aclnnBatchMatmulQuant)

/* Grouped (mixture-of-experts) forms -- replace aclnn_ops.h:2023-2036 (cuda/src/ops/matmul.cu:1195-1202,
 * 1402-1413).  weight [K,N]: the group list is accepted and ignored, as in the reference (one group over all
 * rows).  weight [E,K,N]: the group list holds E entries -- rows per group, or their running totals; either
 * way they end at M -- and the rows of group g are multiplied by weight[g] and dequantised with scale[g]
 * (scale [E,N], or [N] shared by all groups).  ...InplaceAdd: out += result. */
#define B200_ACLNN_QMM_GROUPED(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, \
        const aclTensor *scale, const aclIntArray *groupList, aclTensor *out, uint64_t *workspaceSize, \
        aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_QMM_GROUPED(aclnnQuantGroupedMatmulDequant)
B200_ACLNN_QMM_GROUPED(aclnnQuantGroupedMatmulDequantWeightNZ)
B200_ACLNN_QMM_GROUPED(aclnnQuantGroupedMatmulInplaceAdd)

/* Collective-signature names whose communicator the reference ignores: the local W8A8 matmul.
 * comm is an HcclComm (void *).  Replaces aclnn_mc2.h:82-91 (cuda/src/ops/matmul.cu:1294-1302). */
#define B200_ACLNN_QMM_COMM(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *weight, \
        const aclTensor *scale, void *comm, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_QMM_COMM(aclnnAlltoAllQuantMatmul)
B200_ACLNN_QMM_COMM(aclnnQuantMatmulAlltoAll)
B200_ACLNN_QMM_COMM(aclnnAlltoAllvQuantGroupedMatMul)
B200_ACLNN_QMM_COMM(aclnnQuantGroupedMatMulAlltoAllv)
B200_ACLNN_QMM_COMM(aclnnQuantReduceScatter)
B200_ACLNN_QMM_COMM(aclnnQuantMatmulReduceSumWeightNz)

/* Extended form: out = T( float(acc + bias[n]) * scale[n] * pertokenScale[m] ).
 * bias: ACL_INT32 [N] (added to the exact accumulator); pertokenScale: ACL_FLOAT [M];
 * offsetOptional is accepted for signature compatibility and must be null.
 * With scale == null and out of type ACL_INT32 the raw accumulators are written (the bit-exact
 * check; on the reference they sit in the caller's workspace at byte offset N*K, matmul.cu:821). */
ACL_FUNC_VISIBILITY aclnnStatus aclnnQuantMatmulV4ExGetWorkspaceSize(const aclTensor *x1, const aclTensor *x2,
    const aclTensor *scale, const aclTensor *offsetOptional, const aclTensor *pertokenScaleOptional,
    const aclTensor *biasOptional, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnQuantMatmulV4Ex)

/* ---- MX block-scaled matmul ---------------------------------------------------------------------
 * out[M,N] = sum_k self[m,k]*2^(selfScale[m,k/32]-127) * other[k,n]*2^(otherScale[k/32,n]-127)
 * self [M,K], other [K,N]: fp8 e4m3/e5m2 (one byte each) or fp4 e2m1 (two per byte, element 0 =
 * low nibble); the two operands may differ (MXFP8 x MXFP4).  Scales ACL_FLOAT8_E8M0.
 * out: ACL_FLOAT16 / ACL_BF16 / ACL_FLOAT.  All four names run the same native kernels.
 * Replaces include/aclnnop/aclnn_ops.h:1021-1038 (cuda/src/ops/matmul.cu:432-518,538-597,657-730). */
#define B200_ACLNN_MX(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *self, const aclTensor *selfScale, \
        const aclTensor *other, const aclTensor *otherScale, aclTensor *out, \
        uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_MX(aclnnMatmulMxFp8)
B200_ACLNN_MX(aclnnMatmulMxFp8Hw)
B200_ACLNN_MX(aclnnMatmulMxFp4)
B200_ACLNN_MX(aclnnMatmulMxFp4Hw)

/* ---- Weight pre-pack and test-support operators ------------------------------------------------ */
/* Two int8 values in [-8,7] -> one byte (hi<<4 | lo&0xF), low nibble first.
 * Replaces aclnn_ops.h:1790-1791 (cuda/src/ops/conv.cu:588-591,788-794). */
ACL_FUNC_VISIBILITY aclnnStatus aclnnConvertWeightToINT4PackGetWorkspaceSize(const aclTensor *weight, aclTensor *out,
    uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnConvertWeightToINT4Pack)
/* One-time re-layout of a weight into the on-device format its `out` tensor names, and the size query that goes
 * with it.  Replaces aclnn_ops.h:2009-2014 (cuda/src/ops/matmul.cu:1162-1170), where both are identities.
 * An ACL_INT4 weight [K,N] copied into an out tensor of format ACL_FORMAT_FRACTAL_NZ (same view shape [K,N],
 * storage of aclnnCalculateMatmulWeightSizeV2(shape, ACL_INT4) elements) becomes the tile-packed layout the
 * decode kernel streams with contiguous 16 KB copies: blocks of 256 columns x 128 rows, tile-major, padded with
 * zeros.  The aclnnWeightQuantBatchMatmul* entry points recognise the format on the weight tensor (any of the
 * names, not only ...Nz) and give the same bits as on the caller's layout.  Every other case -- other types,
 * ND destination -- is the identity copy of the reference, and aclnnCalculateMatmulWeightSize (no type) the
 * product of the dimensions. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnTransMatmulWeightGetWorkspaceSize(const aclTensor *weight, aclTensor *out,
    uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnTransMatmulWeight)
/* Per-token dynamic int8 quantiser, the producer of x1 and pertokenScale for the W8A8 matmul:
 * per row of x [..., D] (ACL_FLOAT, ACL_FLOAT16 or ACL_BF16): scaleOut = max|x| / 127 (1 for a zero row,
 * ACL_FLOAT, one per row), out = clamp(rint(x * (1 / scaleOut)), -128, 127) as ACL_INT8.
 * Replaces aclnn_ops.h:1076-1095 (cuda/src/ops/quant.cu:37-49,99-111). */
#define B200_ACLNN_DYNQUANT(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, aclTensor *out, aclTensor *scaleOut, \
        uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_DYNQUANT(aclnnDynamicQuant)
B200_ACLNN_DYNQUANT(aclnnDynamicQuantV2)
B200_ACLNN_DYNQUANT(aclnnDynamicQuantV3)
B200_ACLNN_DYNQUANT(aclnnDynamicQuantV4)

/* SwiGLU fused with the per-token quantiser, the step between a gate/up projection and a W8A8 down
 * projection: x [..., 2 D] (ACL_FLOAT, ACL_FLOAT16 or ACL_BF16) holds a = x[..., :D] and b = x[..., D:];
 * g = a / (1 + exp(-a)) * b in fp32; scaleOut = max|g| / 127 (1 for a zero row; ACL_FLOAT, one per row),
 * out [..., D] = clamp(rint(g * (1 / scaleOut)), -127, 127) as ACL_INT8.
 * Replaces aclnn_ops.h:1275-1278 (cuda/src/ops/glu_ext.cu:89-103,118-141). */
B200_ACLNN_DYNQUANT(aclnnSwiGluQuant)
B200_ACLNN_DYNQUANT(aclnnSwiGluQuantV2)
/* The same behind an optional per-row dequant scale (ACL_FLOAT, one per row, or NULL): a and b are
 * multiplied by dequantScale[row] before the SwiGLU.
 * Replaces aclnnDequantSwigluQuant[V2] of aclnn_ops.h (cuda/src/ops/norm_ext.cu:1354-1369,1416-1432). */
#define B200_ACLNN_DEQSWIGLUQUANT(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, const aclTensor *dequantScale, aclTensor *out, \
        aclTensor *scaleOut, uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_DEQSWIGLUQUANT(aclnnDequantSwigluQuant)
B200_ACLNN_DEQSWIGLUQUANT(aclnnDequantSwigluQuantV2)

/* Residual add + RMS norm, the tail of the all-reduce matmuls: v = x + residual in fp32,
 * residualSum = T(v), y = T(float(residualSum) * rsqrt(mean(v^2) + eps) * gamma) per row of the last
 * dimension; x, residual, y, residualSum of one type (ACL_FLOAT, ACL_FLOAT16, ACL_BF16), gamma [D] or NULL.
 * residualSum may alias residual and y may alias x.
 * Replaces aclnnAddRmsNorm of aclnn_ops.h (cuda/src/ops/norm_ext.cu:123-139,233-247). */
ACL_FUNC_VISIBILITY aclnnStatus aclnnAddRmsNormGetWorkspaceSize(const aclTensor *x, const aclTensor *residual,
    const aclTensor *gamma, double eps, aclTensor *y, aclTensor *residualSum, uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnAddRmsNorm)

/* Block-wise dynamic int8 quantiser with power-of-two scales: per block of blockSize consecutive elements
 * scaleOut = 2^ceil(log2(max|x| / 127)) (1 for a zero block; ACL_FLOAT, one per block),
 * out = clamp(rint(x * (1 / scaleOut)), -128, 127) as ACL_INT8.
 * Replaces aclnn_ops.h:1481-1484 (cuda/src/ops/quant.cu:380-389,496-514). */
#define B200_ACLNN_MXQUANT(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *x, int64_t blockSize, aclTensor *out, \
        aclTensor *scaleOut, uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_MXQUANT(aclnnDynamicMxQuant)
B200_ACLNN_MXQUANT(aclnnDynamicMxQuantV2)

/* fp32 scale (+ optional fp32 offset) -> ACL_INT64 quant parameter: low 32 bits = bits of the scale,
 * high 32 bits = offset rounded to the nearest int32.  Replaces aclnn_ops.h:1730-1735
 * (cuda/src/ops/quant.cu:572-576,657-673). */
#define B200_ACLNN_QPARAM(NAME) \
    ACL_FUNC_VISIBILITY aclnnStatus NAME##GetWorkspaceSize(const aclTensor *scale, const aclTensor *offset, \
        aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor); \
    B200_ACLNN_RUN(NAME)
B200_ACLNN_QPARAM(aclnnTransQuantParam)
B200_ACLNN_QPARAM(aclnnTransQuantParamV2)
B200_ACLNN_QPARAM(aclnnTransQuantParamV3)
ACL_FUNC_VISIBILITY aclnnStatus aclnnCalculateMatmulWeightSizeGetWorkspaceSize(const aclIntArray *weightShape, aclTensor *out,
    uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnCalculateMatmulWeightSize)
ACL_FUNC_VISIBILITY aclnnStatus aclnnCalculateMatmulWeightSizeV2GetWorkspaceSize(const aclIntArray *weightShape, int64_t dtype,
    aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnCalculateMatmulWeightSizeV2)
/* Element-wise cast between ACL_FLOAT and {fp16, bf16, fp8 e4m3/e5m2, fp4 e2m1, int8, int32}; the MX
 * tests build their operands with it.  Replaces aclnn_ops.h:116-118 (cuda/src/ops/cast.cu:157-202). */
ACL_FUNC_VISIBILITY aclnnStatus aclnnCastGetWorkspaceSize(const aclTensor *self, aclDataType dtype, aclTensor *out,
    uint64_t *workspaceSize, aclOpExecutor **executor);
B200_ACLNN_RUN(aclnnCast)

/* Decode-shaped weight-only matmul in ONE call that allocates nothing and takes no workspace.
 * It has no counterpart in the reference.  It exists for programs whose decode path was written
 * against the reference's "0 workspace bytes for M <= 16" (cuda/src/ops/matmul.cu:773-774) and that run
 * where device memory can no longer be requested (arena fixed at start-up, no allocation calls in the
 * serving loop): the split-K partial sums live in a 2 MiB array inside the library, held by every GPU
 * that loads it.
 *   out[m,n] = x[m,k] @ ((weight - offset) * scale) + bias, same semantics and layouts as
 *   aclnnWeightQuantBatchMatmulV2Ex; x/scale/offset/bias/out are all of xType (ACL_FLOAT16, ACL_BF16 or
 *   ACL_FLOAT), weightType is ACL_INT8 or ACL_INT4, antiquantGroupSize 0 = per-channel [N] scales.
 * Limits: M <= 4, N a multiple of 32, and split * M * N partial sums must fit the 2 MiB (larger
 * problems return 161002 with a message on stderr).  The weight pointer must be 16-byte aligned
 * (8-byte for M = 3..4): the kernel reads the packed weights with vector loads, and a pointer off that
 * boundary is refused with 361001 before anything is launched.  The first call on each device looks up
 * the array's device address, and the first call of each (weightType, M = 1 | 2 | 3..4) form sets that
 * kernel's attributes: warm up every form you will use once per device before any stream capture.  First
 * calls from two threads may both look the address up (they store the same value).  All calls share
 * the array: calls whose kernels could overlap on the GPU must be serialised by the caller. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnB200WeightQuantMatmulNoAlloc(const void *x, const void *weight,
    const void *antiquantScale, const void *antiquantOffsetOptional, const void *biasOptional, void *out,
    int64_t m, int64_t k, int64_t n, int64_t antiquantGroupSize, aclDataType xType, aclDataType weightType,
    aclrtStream stream);

/* Plans of composite operators that live in another library (the all-reduce matmuls of libhccl.so;
 * no counterpart in the reference, which keeps such state in process-wide maps, cuda/src/ops/mc2_ext.cu:17).
 * aclnnB200CreateWrapperExecutor returns a real executor that owns `payload`: aclDestroyAclOpExecutor
 * calls payload_free(payload), and the plain execute entries refuse such a plan with 161002.
 * aclnnB200WrapperPayload returns the payload (NULL for any other executor); with release != 0 the
 * executor gives up ownership of it. */
ACL_FUNC_VISIBILITY aclOpExecutor *aclnnB200CreateWrapperExecutor(void *payload, void (*payload_free)(void *));
/* A view of rows [firstRow, firstRow + rows) of the leading dimension of `tensor` over the same buffer (the
 * composite operators cut their work into row chunks with it; the public meta API has no stride getters).
 * NULL for a range outside the tensor.  Destroyed with aclDestroyTensor. */
ACL_FUNC_VISIBILITY aclTensor *aclnnB200CreateRowSlice(const aclTensor *tensor, int64_t firstRow, int64_t rows);
/* The dense tensor-core kernels are persistent, one CTA per SM; a kernel enqueued on another stream (a
 * collective) could then not start before they finish.  After aclnnB200ReserveSms(n) the plans the CALLING
 * THREAD makes (both phases must see the same value) leave n SMs unused; 0 restores the default.  Used by the
 * all-reduce matmuls of libhccl.so around their row chunks. */
ACL_FUNC_VISIBILITY void aclnnB200ReserveSms(int32_t sms);
/* Gathering epilogue of the weight-only decode kernel (used by aclnnB200WeightQuantMatmulAllGather of libhccl.so; no
 * counterpart in the reference).  While set, the CALLING THREAD's weight-only matmuls of up to 16 rows also store every
 * output row into the receive windows of the other GPUs of a column-partitioned layer, as 8-byte packets {two 16-bit
 * outputs, the call's number}: peer[i] is GPU i's window as this process sees it, two receive buffers of buf_bytes
 * each (they alternate by call), calls the device counter of completed calls.  Both phases of a call must see the same
 * setting; NULL clears.  aclnnB200DecodeGatherConsumed: 1 if the thread's last launch took the gathering form. */
typedef struct aclnnB200DecodeGather {
    void *peer[8];
    const unsigned long long *calls;
    uint32_t nranks, rank;
    uint64_t buf_bytes;
    uint32_t f32, reserved; /* f32 != 0: packets {one fp32 output, number}, stored into the own window too (partial results
                             * that a receiver sums: the K-split all-reduce form; no bias allowed) */
} aclnnB200DecodeGather;
ACL_FUNC_VISIBILITY void aclnnB200SetDecodeGather(const aclnnB200DecodeGather *gather);
ACL_FUNC_VISIBILITY int32_t aclnnB200DecodeGatherConsumed(void);
ACL_FUNC_VISIBILITY void *aclnnB200WrapperPayload(aclOpExecutor *executor, int release);

/* Diagnostics (no counterpart in the reference): number of kernels this library has launched in the
 * calling process so far.  Benchmarks use the difference around a timed region. */
ACL_FUNC_VISIBILITY uint64_t aclnnB200KernelLaunchCount(void);
/* Diagnostics (no counterpart in the reference): 0, or the code of the first bounded wait inside a
 * tensor-core kernel that gave up on the current device.  Synchronises the device. */
ACL_FUNC_VISIBILITY uint32_t aclnnB200DeviceStatus(void);
/* Failure handling (no counterpart in the reference, whose kernels have no waits): every wait inside a
 * kernel of this library is bounded; a wait that runs out makes its kernel return early with undefined
 * results and records a code.  Once aclnnB200DeviceStatus() has reported a non-zero code, every matmul
 * execute call on that device returns ACLNN_ERR_RUNTIME_ERROR (361001) without launching, until
 * aclnnB200ResetDeviceStatus() clears the code.  Synchronises the device. */
ACL_FUNC_VISIBILITY void aclnnB200ResetDeviceStatus(void);

#ifdef __cplusplus
}
#endif
#endif
