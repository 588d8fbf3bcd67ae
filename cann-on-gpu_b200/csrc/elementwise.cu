// Small element-wise kernels around the matmuls: int4 weight pack and dtype casts (test support:
// the MX tests quantise their operands with aclnnCast, reference cuda/src/ops/cast.cu:157-202).
#include <atomic>

#include "device_utils.cuh"

namespace qmm {
namespace {

// out[i] = (in[2i+1] << 4) | (in[2i] & 0xF): low nibble first (reference cuda/src/ops/conv.cu:588-591).
// Each thread packs 8 inputs into one 32-bit word when the tail allows it.
__global__ void int4_pack_kernel(const int8_t *in, uint8_t *out, int64_t n_out) {
    int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n_out) return;
    if (i + 4 <= n_out && (reinterpret_cast<uintptr_t>(in) & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0) {
        uint2 v = *reinterpret_cast<const uint2 *>(in + 2 * i);
        uint32_t lo = v.x & 0x0F0F0F0Fu, hi = v.y & 0x0F0F0F0Fu;  // 4 values each, one per byte
        // bytes (a0,a1,a2,a3) -> (a0|a1<<4, a2|a3<<4)
        uint32_t plo = (lo | (lo >> 4)) & 0x00FF00FFu, phi = (hi | (hi >> 4)) & 0x00FF00FFu;
        uint32_t w = (plo & 0xFF) | ((plo >> 8) & 0xFF00) | ((phi & 0xFF) << 16) | ((phi << 8) & 0xFF000000u);
        *reinterpret_cast<uint32_t *>(out + i) = w;
        return;
    }
    for (int64_t j = i; j < n_out && j < i + 4; ++j)
        out[j] = (uint8_t)(((in[2 * j + 1] & 0xF) << 4) | (in[2 * j] & 0xF));
}

// fp4 e2m1 encode with the reference's magnitude boundaries (cuda/src/ops/subfp.cuh:44,62-70):
// normal values round to nearest even, the two sub-1.0 boundaries are the Ascend library's;
// NaN -> +0, out of range saturates to +-6.
__device__ __forceinline__ uint32_t float_to_e2m1(float x) {
    const float bound[7] = {0.4375f, 0.875f, 1.25000012f, 1.75f, 2.50000024f, 3.5f, 5.00000048f};
    if (x != x) return 0;
    float ax = fabsf(x);
    uint32_t c = 0;
#pragma unroll
    for (int i = 0; i < 7; ++i) c += ax >= bound[i] ? 1u : 0u;
    return (__float_as_uint(x) >> 31) ? (c | 8u) : c;
}

__device__ __forceinline__ uint32_t float_to_code(float v, int t) {
    if (t == ET_E4M3) return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    if (t == ET_E5M2) return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2);
    return float_to_e2m1(v);
}

// One thread per output byte for sub-byte destinations (two elements), per element otherwise.
__global__ void cast_kernel(const void *in, int in_type, void *out, int out_type, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (out_type == ET_E2M1) {
        if (2 * i >= n) return;
        uint32_t lo = float_to_code(load_as_float(in, in_type, 2 * i), ET_E2M1);
        uint32_t hi = 2 * i + 1 < n ? float_to_code(load_as_float(in, in_type, 2 * i + 1), ET_E2M1) : 0u;
        ((uint8_t *)out)[i] = (uint8_t)(lo | (hi << 4));
        return;
    }
    if (i >= n) return;
    float v = load_as_float(in, in_type, i);
    if (out_type == ET_E4M3 || out_type == ET_E5M2) ((uint8_t *)out)[i] = (uint8_t)float_to_code(v, out_type);
    else store_from_float(out, out_type, i, v);
}

__global__ void fill_i64_kernel(int64_t *out, int64_t value) { *out = value; }

}  // namespace

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// Quant parameter word: low 32 bits = the fp32 bits of the scale, high 32 bits = the offset rounded to
// the nearest int32 (0 without an offset).  Reference: cuda/src/ops/quant.cu:572-576.
__global__ void qparam_kernel(const float *scale, const float *offset, int64_t *out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t s = __float_as_uint(scale[i]);
    const uint32_t o = offset ? (uint32_t)__float2int_rn(offset[i]) : 0u;
    out[i] = (int64_t)(((uint64_t)o << 32) | (uint64_t)s);
}

cudaError_t launch_qparam(const float *scale, const float *offset, int64_t *out, int64_t n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    qparam_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(scale, offset, out, n);
    count_launch();
    return cudaGetLastError();
}

// Residual add + RMS norm, the tail of the all-reduce matmuls (cuda/src/ops/norm_ext.cu:123-139):
// v = x + residual in fp32; residual_sum = T(v); y = T(float(residual_sum) * rsqrt(mean(v^2) + eps) * gamma).
// One CTA per row.  The second pass reads residual_sum back, like the reference, so residual_sum may
// alias residual and y may alias x.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const void *x, const void *res, const void *gamma, int type, int gamma_type,
                                                          void *ysum, void *y, int64_t D, float eps) {
    __shared__ float sh[8];
    const int64_t base = (int64_t)blockIdx.x * D;
    float ss = 0.f;
    for (int64_t d = threadIdx.x; d < D; d += 256) {
        const float v = load_as_float(x, type, base + d) + load_as_float(res, type, base + d);
        store_from_float(ysum, type, base + d, v);
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += sh[w];
    const float inv = rsqrtf(tot / (float)D + eps);
    for (int64_t d = threadIdx.x; d < D; d += 256) {
        const float g = gamma ? load_as_float(gamma, gamma_type, d) : 1.f;
        store_from_float(y, type, base + d, load_as_float(ysum, type, base + d) * inv * g);
    }
}

cudaError_t launch_add_rmsnorm(const void *x, const void *res, const void *gamma, int type, int gamma_type, void *ysum, void *y,
                               int64_t rows, int64_t D, float eps, cudaStream_t s) {
    if (rows <= 0 || D <= 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    add_rmsnorm_kernel<<<(unsigned)rows, 256, 0, s>>>(x, res, gamma, type, gamma_type, ysum, y, D, eps);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_fill_i64(int64_t *out, int64_t value, cudaStream_t s) {
    fill_i64_kernel<<<1, 1, 0, s>>>(out, value);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_int4_pack(const int8_t *in, uint8_t *out, int64_t n_out, cudaStream_t s) {
    if (n_out <= 0) return cudaSuccess;
    int64_t threads = (n_out + 3) / 4;
    int4_pack_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(in, out, n_out);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_cast(const void *in, int in_type, void *out, int out_type, int64_t n, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    int64_t threads = out_type == ET_E2M1 ? (n + 1) / 2 : n;
    cast_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(in, in_type, out, out_type, n);
    count_launch();
    return cudaGetLastError();
}

}  // namespace qmm
