// Dynamic int8 quantisers of activations (per token, block-wise, and SwiGLU fused with per token).
//
// Per-token, the step in front of the W8A8 matmul: for every row of x
//   scale = max|x| / 127 (1 for an all-zero row),  q = clamp(rint(x * (1 / scale)), -128, 127)
// written as int8 plus the fp32 scale per row (which the matmul takes as pertokenScale).
// Same arithmetic, in the same order, as the reference (cuda/src/ops/quant.cu:37-49): the quotient
// is formed as x * (1.f / scale) in fp32 and rounded half-to-even, so results are bit-identical.
//
// HBM-bound: the reference reads x twice (maximum, then quantise); here a row of up to 16384 elements
// stays in registers between the two phases, so x is read once: algorithmic bytes per row
// D * (sizeof(x) + 1) + 4.  One CTA per row, 16-byte loads and 8/16-byte stores.
#include <cstdlib>

#include "kernels.h"
#include "tc_common.cuh"

namespace qmm {
namespace {

constexpr int DQ_THREADS = 256;
constexpr int DQ_VEC = 8;   // elements per 16-byte load of a 16-bit type

__device__ __forceinline__ int8_t quant_i8(float v) {
    const int q = (int)rintf(v);
    return (int8_t)(q < -128 ? -128 : (q > 127 ? 127 : q));
}
// Four 32-bit integers -> four signed bytes, each clamped to [-128, 127], q0 in the lowest byte.  With __float2int_rn in
// front this is quant_i8 of four values: round to nearest even, clamp, NaN -> 0.
__device__ __forceinline__ uint32_t pack4_s8(int q0, int q1, int q2, int q3) {
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(q3), "r"(q2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(q1), "r"(q0), "r"(hi));
    return r;
}

template <int THREADS>
__device__ __forceinline__ float block_max_t(float v, float *sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) m = fmaxf(m, sh[w]);
    return m;
}

__device__ __forceinline__ float block_max(float v, float *sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = 0.f;
#pragma unroll
    for (int w = 0; w < DQ_THREADS / 32; ++w) m = fmaxf(m, sh[w]);
    return m;
}

// 16-bit inputs, D % 8 == 0, D <= THREADS * 8 * CHUNKS: the row lives in registers.
template <bool BF16, int CHUNKS, int THREADS>
__global__ void __launch_bounds__(THREADS) dynquant_row_kernel(const uint16_t *x, int8_t *q, float *scale_out, int64_t D) {
    __shared__ float sh[THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * D;
    uint4 v[CHUNKS];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int64_t d = ((int64_t)c * THREADS + threadIdx.x) * DQ_VEC;
        v[c] = make_uint4(0, 0, 0, 0);
        if (d < D) v[c] = __ldg(reinterpret_cast<const uint4 *>(x + base + d));
        const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            if constexpr (BF16) { lo = __uint_as_float(w[i] << 16); hi = __uint_as_float(w[i] & 0xFFFF0000u); }
            else { lo = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xFFFFu))); hi = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16))); }
            amax = fmaxf(amax, fmaxf(fabsf(lo), fabsf(hi)));
        }
    }
    const float m = block_max_t<THREADS>(amax, sh);
    const float scale = m == 0.f ? 1.f : m / 127.f;
    if (threadIdx.x == 0) scale_out[blockIdx.x] = scale;
    const float inv = 1.f / scale;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int64_t d = ((int64_t)c * THREADS + threadIdx.x) * DQ_VEC;
        if (d >= D) continue;
        const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
        int qi[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            if constexpr (BF16) { lo = __uint_as_float(w[i] << 16); hi = __uint_as_float(w[i] & 0xFFFF0000u); }
            else { lo = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xFFFFu))); hi = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16))); }
            qi[2 * i] = __float2int_rn(lo * inv);
            qi[2 * i + 1] = __float2int_rn(hi * inv);
        }
        *reinterpret_cast<uint2 *>(q + base + d) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
    }
}

// Any type, any D: two passes over the row (the second one hits L2).
__global__ void __launch_bounds__(DQ_THREADS) dynquant_generic_kernel(const void *x, int x_type, int8_t *q, float *scale_out, int64_t D) {
    __shared__ float sh[DQ_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * D;
    float amax = 0.f;
    for (int64_t d = threadIdx.x; d < D; d += DQ_THREADS) amax = fmaxf(amax, fabsf(load_as_float(x, x_type, base + d)));
    const float m = block_max(amax, sh);
    const float scale = m == 0.f ? 1.f : m / 127.f;
    if (threadIdx.x == 0) scale_out[blockIdx.x] = scale;
    const float inv = 1.f / scale;
    for (int64_t d = threadIdx.x; d < D; d += DQ_THREADS) q[base + d] = quant_i8(load_as_float(x, x_type, base + d) * inv);
}

// ---- block-wise power-of-two scales ("MX-style" int8): per block of `blk` consecutive elements
//   scale = 2^ceil(log2(max|x| / 127)) (1 for an all-zero block),  q = clamp(rint(x * (1 / scale)))
// with the reference's expression exp2f(ceilf(log2f(m / 127.f))) evaluated by the same device functions
// (cuda/src/ops/quant.cu:380-389), so scales and codes are bit-identical to it.
__device__ __forceinline__ float mx_block_scale(float m) { return m > 0.f ? exp2f(ceilf(log2f(m / 127.f))) : 1.f; }

// 16-bit inputs, blk = 8 * LPB with LPB (lanes per block) in {4, 8, 16, 32}: a lane holds 8 elements
// (one 16-byte load), a block's maximum is LPB-lane butterfly, 8-byte stores of the codes.
template <bool BF16, int LPB>
__global__ void __launch_bounds__(256) mxquant_vec_kernel(const uint16_t *x, int8_t *q, float *scale_out, int64_t n) {
    const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    const bool in = i0 < n;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (in) v = __ldg(reinterpret_cast<const uint4 *>(x + i0));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8], amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
        else { f[2 * i] = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xFFFFu))); f[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16))); }
        amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
    }
#pragma unroll
    for (int o = LPB / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = mx_block_scale(amax);
    if (in && (threadIdx.x & (LPB - 1)) == 0) scale_out[i0 / (8 * LPB)] = sc;
    const float inv = 1.f / sc;
    int qi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qi[i] = __float2int_rn(f[i] * inv);
    if (in) *reinterpret_cast<uint2 *>(q + i0) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
}

// Any type, any block size: one CTA per block.
__global__ void __launch_bounds__(DQ_THREADS) mxquant_generic_kernel(const void *x, int x_type, int8_t *q, float *scale_out, int64_t blk) {
    __shared__ float sh[DQ_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * blk;
    float amax = 0.f;
    for (int64_t d = threadIdx.x; d < blk; d += DQ_THREADS) amax = fmaxf(amax, fabsf(load_as_float(x, x_type, base + d)));
    const float sc = mx_block_scale(block_max(amax, sh));
    if (threadIdx.x == 0) scale_out[blockIdx.x] = sc;
    const float inv = 1.f / sc;
    for (int64_t d = threadIdx.x; d < blk; d += DQ_THREADS) q[base + d] = quant_i8(load_as_float(x, x_type, base + d) * inv);
}

// ---- SwiGLU fused with the per-token quantiser: the step between the gate/up projection and a W8A8
// down projection.  Row layout [a (D) | b (D)]; g = a / (1 + exp(-a)) * b in fp32, evaluated with the
// reference's expression (cuda/src/ops/glu_ext.cu:89-103); scale = max|g| / 127 (1 for an all-zero
// row), q = clamp(rint(g * (1 / scale)), -127, 127).  With a per-row dequant scale dq (DequantSwigluQuant,
// cuda/src/ops/norm_ext.cu:1354-1369) a and b are first multiplied by dq[row].  The reference computes g twice (maximum, then
// quantise); here a row of up to 16384 outputs keeps g in registers: one read of 2 D inputs, one
// write of D codes.
__device__ __forceinline__ float swiglu_of(float a, float b) { return a / (1.f + expf(-a)) * b; }
__device__ __forceinline__ int8_t quant_i8_sym(float v) {
    const int q = __float2int_rn(v);
    return (int8_t)(q < -127 ? -127 : (q > 127 ? 127 : q));
}
template <bool BF16> __device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
        else { f[2 * i] = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xFFFFu))); f[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16))); }
    }
}

// 16-bit inputs, D % 8 == 0, D <= THREADS * 8 * CHUNKS.  Long rows use 512 threads with at most four
// chunks each: the arithmetic per element (expf, an IEEE division) needs the occupancy more than the
// per-token quantiser does.
template <bool BF16, int CHUNKS, int THREADS>
__global__ void __launch_bounds__(THREADS) swigluquant_row_kernel(const uint16_t *x, const float *dq, int8_t *q, float *scale_out, int64_t D) {
    __shared__ float sh[THREADS / 32];
    const float scl = dq ? __ldg(dq + blockIdx.x) : 1.f;   // optional per-row dequant scale (x * 1 is exact)
    const int64_t ib = (int64_t)blockIdx.x * 2 * D, ob = (int64_t)blockIdx.x * D;
    float g[CHUNKS][8];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int64_t d = ((int64_t)c * THREADS + threadIdx.x) * DQ_VEC;
        uint4 va = make_uint4(0, 0, 0, 0), vb = make_uint4(0, 0, 0, 0);
        if (d < D) {
            va = __ldg(reinterpret_cast<const uint4 *>(x + ib + d));
            vb = __ldg(reinterpret_cast<const uint4 *>(x + ib + D + d));
        }
        float fa[8], fb[8];
        unpack8<BF16>(va, fa);
        unpack8<BF16>(vb, fb);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            g[c][i] = swiglu_of(fa[i] * scl, fb[i] * scl);      // 0 beyond the row: silu(0) * 0
            amax = fmaxf(amax, fabsf(g[c][i]));
        }
    }
    const float m = block_max_t<THREADS>(amax, sh);
    const float scale = m > 0.f ? m / 127.f : 1.f;
    if (threadIdx.x == 0) scale_out[blockIdx.x] = scale;
    const float inv = 1.f / scale;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int64_t d = ((int64_t)c * THREADS + threadIdx.x) * DQ_VEC;
        if (d >= D) continue;
        uint32_t o[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i >> 2] |= (uint32_t)(uint8_t)quant_i8_sym(g[c][i] * inv) << (8 * (i & 3));
        *reinterpret_cast<uint2 *>(q + ob + d) = make_uint2(o[0], o[1]);
    }
}

// Many long rows: persistent CTAs that stage their rows through a ring of shared-memory slots.  One thread keeps
// SGQ_STAGES rows in flight with bulk copies (one copy per row: a and b halves are contiguous), so the loads of the
// following rows overlap the arithmetic of this one (expf and an IEEE division per element: the issue slots are busy
// longer than the row's bytes occupy HBM) instead of alternating with it as in the one-row-per-CTA kernel
// ([2048, 28672] bf16: 57.5 -> 43.2 us).  The block
// size is chosen so that CHUNKS * blockDim.x * 8 covers D with no idle lanes where D allows (14336 -> 896 threads).
// A slot is refilled right after the row-maximum barrier, when every thread has its part of the row in registers.
__device__ __forceinline__ void bulk_row_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
template <bool BF16, int CHUNKS, int SGQ_STAGES, bool HAS_DQ>
__global__ void __launch_bounds__(1024) swigluquant_staged_kernel(const uint16_t *x, const float *dq, int8_t *q, float *scale_out,
                                                                  int64_t rows, int64_t D) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t full[SGQ_STAGES];
    __shared__ float sh[2][32];
    __shared__ int abort_flag;
    const int tid = threadIdx.x, T = blockDim.x, nwarps = T >> 5;
    const uint32_t row_bytes = (uint32_t)(D * 4);       // 2 D elements of 2 bytes
    const uint32_t ring0 = smem_u32(ring);
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < SGQ_STAGES; ++s) mbar_init(smem_u32(&full[s]), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < SGQ_STAGES; ++s) {
            const int64_t r = blockIdx.x + (int64_t)s * gridDim.x;
            if (r < rows) {
                mbar_expect_tx(smem_u32(&full[s]), row_bytes);
                bulk_row_g2s(ring0 + s * row_bytes, x + r * 2 * D, row_bytes, smem_u32(&full[s]));
            }
        }
    }
    int slot = 0;
    uint32_t parity = 0, it = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
        const bool ok = mbar_wait(smem_u32(&full[slot]), parity, &abort_flag, 0x510u);
        const float scl = HAS_DQ ? __ldg(dq + row) : 1.f;
        const uint8_t *sa = ring + (size_t)slot * row_bytes;
        float g[CHUNKS][8];
        float amax = 0.f;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int64_t d = ((int64_t)c * T + tid) * DQ_VEC;
            uint4 va = make_uint4(0, 0, 0, 0), vb = make_uint4(0, 0, 0, 0);
            if (ok && d < D) {
                va = *reinterpret_cast<const uint4 *>(sa + d * 2);
                vb = *reinterpret_cast<const uint4 *>(sa + (D + d) * 2);
            }
            float fa[8], fb[8];
            unpack8<BF16>(va, fa);
            unpack8<BF16>(vb, fb);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                g[c][i] = HAS_DQ ? swiglu_of(fa[i] * scl, fb[i] * scl) : swiglu_of(fa[i], fb[i]);
                amax = fmaxf(amax, fabsf(g[c][i]));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float *shp = sh[it & 1];
        if ((tid & 31) == 0) shp[tid >> 5] = amax;
        // the barrier also says that the slot has been read by everyone, and carries a wait that gave up to all threads
        if (__syncthreads_or(!ok)) break;
        if (tid == 0) {
            const int64_t nr = row + (int64_t)SGQ_STAGES * gridDim.x;
            if (nr < rows) {
                fence_proxy_async();
                mbar_expect_tx(smem_u32(&full[slot]), row_bytes);
                bulk_row_g2s(ring0 + slot * row_bytes, x + nr * 2 * D, row_bytes, smem_u32(&full[slot]));
            }
        }
        float m = shp[(tid & 31) < nwarps ? (tid & 31) : 0];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float scale = m > 0.f ? m / 127.f : 1.f;
        if (tid == 0) scale_out[row] = scale;
        const float inv = 1.f / scale;
        const int64_t ob = row * D;
        // With a row maximum in the normal range |g * inv| <= 127 (1 + 2^-22), so the conversion needs no clamp and the
        // codes can be packed by the saturating pack instruction (a NaN converts to 0 either way); a row whose maximum is
        // so small that max / 127 leaves the normal range takes the clamping form.
        const bool plain = m >= 1e-30f && m <= 3e38f;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int64_t d = ((int64_t)c * T + tid) * DQ_VEC;
            if (d >= D) continue;
            uint32_t o[2] = {0, 0};
            if (plain) {
#pragma unroll
                for (int w = 0; w < 2; ++w)
                    o[w] = pack4_s8(__float2int_rn(g[c][4 * w] * inv), __float2int_rn(g[c][4 * w + 1] * inv),
                                    __float2int_rn(g[c][4 * w + 2] * inv), __float2int_rn(g[c][4 * w + 3] * inv));
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i >> 2] |= (uint32_t)(uint8_t)quant_i8_sym(g[c][i] * inv) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2 *>(q + ob + d) = make_uint2(o[0], o[1]);
        }
        if (++slot == SGQ_STAGES) { slot = 0; parity ^= 1u; }
    }
}

int dq_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!sms[dev]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n > 0 ? n : 1;
    }
    return sms[dev];
}

template <bool BF16, int CHUNKS, int STAGES, bool HAS_DQ>
cudaError_t launch_staged(const uint16_t *x, const float *dq, int8_t *q, float *scale_out, int64_t rows, int64_t D, int threads, cudaStream_t s) {
    auto kernel = swigluquant_staged_kernel<BF16, CHUNKS, STAGES, HAS_DQ>;
    const size_t smem = (size_t)STAGES * D * 4;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    int per_sm = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    if (err != cudaSuccess) return err;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    const int64_t grid = std::min<int64_t>(rows, (int64_t)dq_sm_count() * per_sm);
    kernel<<<(unsigned)grid, threads, smem, s>>>(x, dq, q, scale_out, rows, D);
    return cudaGetLastError();
}

// Any type, any D: g is evaluated twice, the second read of the row hits L2.
__global__ void __launch_bounds__(DQ_THREADS) swigluquant_generic_kernel(const void *x, int x_type, const float *dq, int8_t *q, float *scale_out, int64_t D) {
    __shared__ float sh[DQ_THREADS / 32];
    const float scl = dq ? __ldg(dq + blockIdx.x) : 1.f;
    const int64_t ib = (int64_t)blockIdx.x * 2 * D, ob = (int64_t)blockIdx.x * D;
    float amax = 0.f;
    for (int64_t d = threadIdx.x; d < D; d += DQ_THREADS)
        amax = fmaxf(amax, fabsf(swiglu_of(load_as_float(x, x_type, ib + d) * scl, load_as_float(x, x_type, ib + D + d) * scl)));
    const float m = block_max(amax, sh);
    const float scale = m > 0.f ? m / 127.f : 1.f;
    if (threadIdx.x == 0) scale_out[blockIdx.x] = scale;
    const float inv = 1.f / scale;
    for (int64_t d = threadIdx.x; d < D; d += DQ_THREADS)
        q[ob + d] = quant_i8_sym(swiglu_of(load_as_float(x, x_type, ib + d) * scl, load_as_float(x, x_type, ib + D + d) * scl) * inv);
}

}  // namespace

cudaError_t launch_swiglu_quant(const void *x, int x_type, const float *dq, int8_t *q, float *scale_out, int64_t rows, int64_t D,
                                cudaStream_t s) {
    if (rows <= 0 || D <= 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    const bool vec = (x_type == ET_BF16 || x_type == ET_F16) && D % DQ_VEC == 0 && D <= (int64_t)512 * DQ_VEC * 4 &&
                     (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    const unsigned g = (unsigned)rows;
    const uint16_t *x16 = static_cast<const uint16_t *>(x);
    const int64_t per = (int64_t)DQ_THREADS * DQ_VEC;
    const bool bf = x_type == ET_BF16;
#define SGQ(C, T) do { if (bf) swigluquant_row_kernel<true, C, T><<<g, T, 0, s>>>(x16, dq, q, scale_out, D); \
                       else swigluquant_row_kernel<false, C, T><<<g, T, 0, s>>>(x16, dq, q, scale_out, D); } while (0)
    // rows long enough that the arithmetic matters, and several rows per SM: the staged persistent form
    static const bool staged_on = [] { const char *e = std::getenv("B200_QMM_SGQ_STAGED"); return !e || std::atoi(e) != 0; }();
    if (vec && staged_on && D >= 1024 && rows >= 2 * (int64_t)dq_sm_count()) {
        // one chunk of 8 elements per thread for rows of up to 8192 elements, two above; three ring slots.  (Four chunks with
        // one or two slots, two CTAs per SM, measured the same: the kernel is bound by instruction issue, 43 instructions per
        // element of which 4 on the quarter-rate pipe, not by how the copies overlap.)
        const int64_t vectors = D / DQ_VEC;
        const int chunks = vectors <= 1024 ? 1 : 2;
        const int threads = (int)(((vectors + chunks - 1) / chunks + 31) / 32 * 32);
        cudaError_t err;
#define SGS(B, C) (dq ? launch_staged<B, C, 3, true>(x16, dq, q, scale_out, rows, D, threads, s) \
                      : launch_staged<B, C, 3, false>(x16, dq, q, scale_out, rows, D, threads, s))
        if (chunks == 1) err = bf ? SGS(true, 1) : SGS(false, 1);
        else err = bf ? SGS(true, 2) : SGS(false, 2);
#undef SGS
        if (err != cudaSuccess) return err;
        count_launch();
        return cudaSuccess;
    }
    if (!vec) swigluquant_generic_kernel<<<g, DQ_THREADS, 0, s>>>(x, x_type, dq, q, scale_out, D);
    else if (D <= per) SGQ(1, 256);
    else if (D <= per * 2) SGQ(2, 256);
    else if (D <= per * 4) SGQ(2, 512);
    else SGQ(4, 512);
#undef SGQ
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_dynamic_mx_quant(const void *x, int x_type, int8_t *q, float *scale_out, int64_t nblocks, int64_t blk, cudaStream_t s) {
    if (nblocks <= 0 || blk <= 0) return cudaSuccess;
    const int64_t n = nblocks * blk;
    const bool vec = (x_type == ET_BF16 || x_type == ET_F16) && (blk == 32 || blk == 64 || blk == 128 || blk == 256) &&
                     (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    if (vec) {
        const unsigned g = (unsigned)((n / 8 + 255) / 256);
        const uint16_t *x16 = static_cast<const uint16_t *>(x);
        const bool bf = x_type == ET_BF16;
#define MXQ(LPB) do { if (bf) mxquant_vec_kernel<true, LPB><<<g, 256, 0, s>>>(x16, q, scale_out, n); \
                      else mxquant_vec_kernel<false, LPB><<<g, 256, 0, s>>>(x16, q, scale_out, n); } while (0)
        switch (blk) { case 32: MXQ(4); break; case 64: MXQ(8); break; case 128: MXQ(16); break; default: MXQ(32); break; }
#undef MXQ
    } else {
        if (nblocks > 0x7fffffffLL) return cudaErrorInvalidValue;
        mxquant_generic_kernel<<<(unsigned)nblocks, DQ_THREADS, 0, s>>>(x, x_type, q, scale_out, blk);
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_dynamic_quant(const void *x, int x_type, int8_t *q, float *scale_out, int64_t rows, int64_t D, cudaStream_t s) {
    if (rows <= 0 || D <= 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    const bool vec = (x_type == ET_BF16 || x_type == ET_F16) && D % DQ_VEC == 0 &&
                     (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    const unsigned g = (unsigned)rows;
    const uint16_t *x16 = static_cast<const uint16_t *>(x);
    const int64_t per = (int64_t)DQ_THREADS * DQ_VEC;
    const bool bf = x_type == ET_BF16;
#define DQ(C, T) do { if (bf) dynquant_row_kernel<true, C, T><<<g, T, 0, s>>>(x16, q, scale_out, D); \
                      else dynquant_row_kernel<false, C, T><<<g, T, 0, s>>>(x16, q, scale_out, D); } while (0)
    // rows of up to 4096 elements run 128-thread CTAs: more of them per SM and a shorter tail
    // ([4096,4096] bf16: 11.4 -> 10.1 us)
    if (vec && D <= per / 2) {
        DQ(1, 128);
    } else if (vec && D <= per * 1) {
        DQ(1, 256);
    } else if (vec && D <= per * 2) {
        DQ(4, 128);
    } else if (vec && D <= per * 4) {
        DQ(4, 256);
    } else if (vec && D <= per * 8) {
        DQ(8, 256);
#undef DQ
    } else {
        dynquant_generic_kernel<<<g, DQ_THREADS, 0, s>>>(x, x_type, q, scale_out, D);
    }
    count_launch();
    return cudaGetLastError();
}

unsigned int dynquant_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    return v;
}
void dynquant_device_status_reset() {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(z));
}

}  // namespace qmm
