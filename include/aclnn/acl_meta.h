/*
 * aclnn/acl_meta.h -- minimal, self-declared subset of the aclnn meta-object header.
 *
 * Opaque tensor / scalar / int-array / executor handles and their lifecycle calls, as used by the
 * quantized-matmul operators and their clients (reference implementation: cuda/src/meta.cu:7-113).
 */
#ifndef B200_ACLNN_ACL_META_H
#define B200_ACLNN_ACL_META_H

#include "acl/acl.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t aclnnStatus;

typedef struct aclTensor aclTensor;
typedef struct aclScalar aclScalar;
typedef struct aclIntArray aclIntArray;
typedef struct aclTensorList aclTensorList;
typedef struct aclOpExecutor aclOpExecutor;

/* Host-only metadata over a caller-owned device buffer (reference: cuda/src/meta.cu:7-25). */
ACL_FUNC_VISIBILITY aclTensor *aclCreateTensor(const int64_t *viewDims, uint64_t viewDimsNum, aclDataType dataType,
                                               const int64_t *stride, int64_t offset, aclFormat format,
                                               const int64_t *storageDims, uint64_t storageDimsNum,
                                               void *tensorData);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyTensor(const aclTensor *tensor);
ACL_FUNC_VISIBILITY aclScalar *aclCreateScalar(void *value, aclDataType dataType);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyScalar(const aclScalar *scalar);
ACL_FUNC_VISIBILITY aclIntArray *aclCreateIntArray(const int64_t *value, uint64_t size);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyIntArray(const aclIntArray *array);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor *executor);

/* Getters (reference: cuda/src/meta.cu:88-113). */
ACL_FUNC_VISIBILITY aclnnStatus aclGetViewShape(const aclTensor *tensor, int64_t **viewDims, uint64_t *viewDimsNum);
ACL_FUNC_VISIBILITY aclnnStatus aclGetDataType(const aclTensor *tensor, aclDataType *dataType);
ACL_FUNC_VISIBILITY aclnnStatus aclGetFormat(const aclTensor *tensor, aclFormat *format);
ACL_FUNC_VISIBILITY aclnnStatus aclGetRawTensorAddr(const aclTensor *tensor, void **addr);
ACL_FUNC_VISIBILITY aclnnStatus aclSetRawTensorAddr(aclTensor *tensor, void *addr);

#ifdef __cplusplus
}
#endif
#endif
