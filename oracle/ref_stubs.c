/* Link-time stand-ins for the six symbols the reference's matmul translation unit references from
 * other translation units (norm, BLAS-extension and collective wrappers).  Nothing on the
 * quantized-matmul path calls them; each returns an error.  Test infrastructure only. */
#include <stdint.h>
#define STUB(name) int name(void) { return 361001; }
STUB(HcclAllGather)
STUB(HcclAllReduce)
STUB(aclnnAddRmsNorm)
STUB(aclnnAddRmsNormGetWorkspaceSize)
STUB(aclnnAddmm)
STUB(aclnnAddmmGetWorkspaceSize)
