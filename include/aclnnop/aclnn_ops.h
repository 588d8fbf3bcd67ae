/*
 * aclnnop/aclnn_ops.h -- umbrella header under the include path the reference's clients use
 * (tests/test_matmul_conv.cpp and tests/test_quant_parity.cpp of the reference include this
 * name).  Only the quantized-matmul family is declared.
 */
#ifndef B200_ACLNN_OPS_H
#define B200_ACLNN_OPS_H
#include "aclnnop/aclnn_quant_matmul.h"
#endif
