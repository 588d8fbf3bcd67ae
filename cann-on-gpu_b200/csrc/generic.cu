// Generic CUDA-core tile kernel for the whole quantized-matmul family.
//
// Role: the bounds-checked path for shapes the fast kernels do not take (K not a multiple of the
// MMA step, odd N, fp32 activations, transposed or batched weights) and the on-device cross-check
// for the tensor-core kernels at sizes a CPU oracle cannot reach.  It is the B200 counterpart of the
// reference's functional fallbacks (cuda/src/ops/matmul.cu:853-858 fp16 fallback of QuantMatmul,
// :1097-1101 k_bmm_quant), with the dequantisation done while the tile is loaded instead of in
// separate passes.
//
// 64x64 output tile per CTA, 256 threads, 4x4 outputs per thread, K step 16 staged in shared
// memory.  W8A8 accumulates exactly in int32; everything else in fp32 in ascending k order.
#include "device_utils.cuh"

namespace qmm {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct GenericParams {
    MatmulArgs p;
};

// Dequantised A element (m,k).
__device__ __forceinline__ float load_a(const MatmulArgs &p, const void *a, int64_t m, int64_t k) {
    float v = load_as_float(a, p.a_type, m * p.K + k);
    if (p.a_scale) v *= e8m0_to_float(p.a_scale[m * (p.K / 32) + k / 32]);
    return v;
}
// Dequantised B element (k,n).
__device__ __forceinline__ float load_b(const MatmulArgs &p, const void *b, int64_t k, int64_t n) {
    int64_t idx = p.b_transposed ? n * p.K + k : k * p.N + n;
    float v = load_as_float(b, p.b_type, idx);
    if (p.b_scale) return v * e8m0_to_float(p.b_scale[(k / 32) * p.N + n]);
    if (p.epilogue == EPI_PLAIN && p.scale) {  // weight-only antiquant: (w - offset) * scale
        int64_t g = k / p.group;
        float off = p.offset ? load_as_float(p.offset, p.sc_type, g * p.N + n) : 0.f;
        v = (v - off) * load_as_float(p.scale, p.sc_type, g * p.N + n);
    }
    return v;
}

template <bool INT_ACC>
__global__ void __launch_bounds__(256) generic_kernel(const GenericParams gp) {
    const MatmulArgs &p = gp.p;
    __shared__ float sa[TK][TM + 1];
    __shared__ float sb[TK][TN + 1];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN, bz = blockIdx.z;
    const char *a = (const char *)p.a + bz * p.a_batch_stride * elem_bits(p.a_type) / 8;
    const char *b = (const char *)p.b + bz * p.b_batch_stride * elem_bits(p.b_type) / 8;
    char *out = (char *)p.out + bz * p.out_batch_stride * elem_bits(p.out_type) / 8;

    float facc[4][4] = {};
    int iacc[4][4] = {};
    for (int64_t k0 = 0; k0 < p.K; k0 += TK) {
        for (int i = tid; i < TM * TK; i += 256) {
            int kk = i % TK, mm = i / TK;
            int64_t m = m0 + mm, k = k0 + kk;
            sa[kk][mm] = (m < p.M && k < p.K) ? load_a(p, a, m, k) : 0.f;
        }
        for (int i = tid; i < TN * TK; i += 256) {
            int nn = i % TN, kk = i / TN;
            int64_t n = n0 + nn, k = k0 + kk;
            sb[kk][nn] = (n < p.N && k < p.K) ? load_b(p, b, k, n) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (INT_ACC) iacc[i][j] += (int)av[i] * (int)bv[j];
                    else facc[i][j] = fmaf(av[i], bv[j], facc[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m >= p.M || n >= p.N) continue;
            int64_t o = m * p.N + n;
            if (p.epilogue == EPI_RAW_I32) { ((int32_t *)out)[o] = iacc[i][j]; continue; }
            float v;
            if (p.epilogue == EPI_DEQ_I32) {
                int acc = iacc[i][j] + (p.bias ? ((const int32_t *)p.bias)[n] : 0);
                v = (float)acc * load_as_float(p.scale, p.sc_type, n);
                if (p.pertoken) v = v * p.pertoken[m];
            } else {
                v = facc[i][j];
                if (p.bias) v += load_as_float(p.bias, p.bias_type, n);
            }
            if (p.accumulate) v = load_as_float(out, p.out_type, o) + round_through(p.out_type, v);
            store_from_float(out, p.out_type, o, v);
        }
}

}  // namespace

cudaError_t launch_generic(const MatmulArgs &p, cudaStream_t s) {
    if (p.M <= 0 || p.N <= 0) return cudaSuccess;
    GenericParams gp{p};
    dim3 grid((unsigned)((p.N + TN - 1) / TN), (unsigned)((p.M + TM - 1) / TM), (unsigned)p.batch);
    if (p.epilogue == EPI_PLAIN) generic_kernel<false><<<grid, 256, 0, s>>>(gp);
    else generic_kernel<true><<<grid, 256, 0, s>>>(gp);
    count_launch();
    return cudaGetLastError();
}

}  // namespace qmm
