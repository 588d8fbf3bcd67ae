// Device-side element codecs shared by the kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cstdint>

#include "kernels.h"

namespace qmm {

// fp4 e2m1 magnitudes {0,.5,1,1.5,2,3,4,6}; bit 3 is the sign.  Same values as the reference's
// decode table (cuda/src/ops/subfp.cuh:18-20) and as the hardware's e2m1.
__device__ __forceinline__ float e2m1_to_float(uint32_t code) {
    // magnitude = (code&7): 0 -> 0, 1 -> 0.5, else (1 + (c&1)/2) * 2^((c>>1)-1)
    uint32_t c = code & 7u;
    float m = c == 0 ? 0.f : (c == 1 ? 0.5f : __uint_as_float(((126u + (c >> 1)) << 23) | ((c & 1u) << 22)));
    return (code & 8u) ? -m : m;
}

// e8m0 block scale 2^(e-127).  e = 0 is the fp32 subnormal 2^-127, e = 255 is NaN.
__device__ __forceinline__ float e8m0_to_float(uint32_t e) {
    return e == 0 ? __uint_as_float(0x00400000u) : (e == 255 ? __uint_as_float(0x7fc00000u) : __uint_as_float(e << 23));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}
__device__ __forceinline__ float e5m2_to_float(uint8_t v) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E5M2)));
}

// int4 element `idx` of a packed buffer: even linear index = low nibble, two's complement.
__device__ __forceinline__ int int4_at(const uint8_t *p, int64_t idx) {
    uint32_t byte = p[idx >> 1];
    int v = (idx & 1) ? (byte >> 4) : (byte & 0xf);
    return v >= 8 ? v - 16 : v;
}

// Element `idx` of a buffer of runtime type `t`, as float (exact for every supported type).
__device__ __forceinline__ float load_as_float(const void *p, int t, int64_t idx) {
    switch (t) {
        case ET_F32: return ((const float *)p)[idx];
        case ET_F16: return __half2float(((const __half *)p)[idx]);
        case ET_BF16: return __bfloat162float(((const __nv_bfloat16 *)p)[idx]);
        case ET_I8: return (float)((const int8_t *)p)[idx];
        case ET_U8: return (float)((const uint8_t *)p)[idx];
        case ET_I32: return (float)((const int32_t *)p)[idx];
        case ET_I4: return (float)int4_at((const uint8_t *)p, idx);
        case ET_E4M3: return e4m3_to_float(((const uint8_t *)p)[idx]);
        case ET_E5M2: return e5m2_to_float(((const uint8_t *)p)[idx]);
        case ET_E2M1: {
            uint32_t byte = ((const uint8_t *)p)[idx >> 1];
            return e2m1_to_float((idx & 1) ? (byte >> 4) : (byte & 0xf));
        }
        case ET_E8M0: return e8m0_to_float(((const uint8_t *)p)[idx]);
    }
    return 0.f;
}

// Round-to-nearest-even store of a float into a buffer of runtime type `t`.
__device__ __forceinline__ void store_from_float(void *p, int t, int64_t idx, float v) {
    switch (t) {
        case ET_F32: ((float *)p)[idx] = v; break;
        case ET_F16: ((__half *)p)[idx] = __float2half_rn(v); break;
        case ET_BF16: ((__nv_bfloat16 *)p)[idx] = __float2bfloat16_rn(v); break;
        case ET_I32: ((int32_t *)p)[idx] = __float2int_rn(v); break;
        case ET_I8: ((int8_t *)p)[idx] = (int8_t)max(-128, min(127, __float2int_rn(v))); break;
        case ET_U8: ((uint8_t *)p)[idx] = (uint8_t)max(0, min(255, __float2int_rn(v))); break;
    }
}

// Value after a round trip through the output type (used by the accumulate-into-out variants,
// which round the product to the output type before adding, like the reference's temp buffer).
__device__ __forceinline__ float round_through(int t, float v) {
    switch (t) {
        case ET_F16: return __half2float(__float2half_rn(v));
        case ET_BF16: return __bfloat162float(__float2bfloat16_rn(v));
    }
    return v;
}

}  // namespace qmm
