// Expand-then-dense path: operands that the tensor core cannot read directly are first expanded to
// bf16 / fp16 in the caller's workspace by HBM-bound streaming kernels, then multiplied by the dense
// tcgen05 kernel (tc.cu).
//
//   * MX block-scaled matmuls: element * 2^(scale-127) is exact in bf16 for fp8 and fp4 elements, so
//     expanding both operands and accumulating in fp32 gives the block-scaled product without any
//     rounding of the operands.  (The reference's functional path does the same through fp16,
//     cuda/src/ops/matmul.cu:153-189,454-483; its native path hands the job to cuBLASLt, :578-596.)
//   * Weight-only matmuls with many rows (prefill): wf = (w - offset) * scale rounded once to the
//     activation type, as the reference does (matmul.cu:733-747,790-795), but without its per-call
//     transposes.  With few rows the fused stream-K kernel (wq_tc.cu) is used instead.
#include <cstdlib>

#include "device_utils.cuh"

namespace qmm {
namespace {

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float a, float b) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    } else {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
}

// Weight-only: out[k][n] = T((w[k][n] - off[g][n]) * scale[g][n]), g = k / group.  One thread expands
// 16 consecutive columns of one row (8 B of int4 or 16 B of int8) and writes 32 B.
template <bool Q4, bool BF16, bool OUT_BF16 = BF16>
__global__ void expand_wq_kernel(const uint8_t *w, const void *scale, const void *offset, int sc_type, uint16_t *out, int K, int N,
                                 int group) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = N / 16;
    if (t >= (int64_t)K * per_row) return;
    const int k = (int)(t / per_row), n0 = (int)(t % per_row) * 16;
    const int g = k / group;
    float v[16];
    if constexpr (Q4) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(w + ((size_t)k * N + n0) / 2));
        const uint32_t words[2] = {raw.x, raw.y};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int nib = (words[i >> 3] >> (4 * (i & 7))) & 0xF;
            v[i] = (float)(nib >= 8 ? nib - 16 : nib);
        }
    } else {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(w + (size_t)k * N + n0));
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = (float)(int8_t)((words[i >> 2] >> (8 * (i & 3))) & 0xFF);
    }
    const size_t srow = (size_t)g * N + n0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float s = load_as_float(scale, sc_type, srow + i);
        const float o = offset ? load_as_float(offset, sc_type, srow + i) : 0.f;
        v[i] = (v[i] - o) * s;
    }
    uint4 o0, o1;
    o0.x = pack2<OUT_BF16>(v[0], v[1]);   o0.y = pack2<OUT_BF16>(v[2], v[3]);   o0.z = pack2<OUT_BF16>(v[4], v[5]);   o0.w = pack2<OUT_BF16>(v[6], v[7]);
    o1.x = pack2<OUT_BF16>(v[8], v[9]);   o1.y = pack2<OUT_BF16>(v[10], v[11]); o1.z = pack2<OUT_BF16>(v[12], v[13]); o1.w = pack2<OUT_BF16>(v[14], v[15]);
    uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)k * N + n0);
    dst[0] = o0;
    dst[1] = o1;
}

// The same expansion written for bandwidth: a lane owns 8 consecutive columns (one 32-bit word of
// int4, or 8 bytes of int8) and walks 4 rows of a 32-row chunk, so the 8 scales and 8 offsets of the
// chunk's group are loaded once (two 16-byte loads) and every output is one 16-byte store; integers
// become floats through the 2^23 mantissa trick instead of conversions.  Same fp32 expression per
// element as above, so the same bits.  Needs 16-bit scales of the output type, N % 8 == 0 and a
// group size that is a multiple of 32 (or per-channel scales).
template <bool Q4, bool BF16, int RPT, bool OUT_BF16 = BF16>   // RPT rows per thread: a block covers 8 * RPT rows of one scale group
__global__ void __launch_bounds__(256) expand_wq_fast_kernel(const uint8_t *w, const uint16_t *scale, const uint16_t *offset,
                                                             uint16_t *out, int K, int N, int group) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int n0 = (blockIdx.x * 32 + lane) * 8;
    const int k0 = blockIdx.y * (8 * RPT);
    if (n0 >= N) return;
    const int g = k0 / group;
    const uint4 sraw = __ldg(reinterpret_cast<const uint4 *>(scale + (size_t)g * N + n0));
    uint4 oraw = make_uint4(0, 0, 0, 0);
    if (offset) oraw = __ldg(reinterpret_cast<const uint4 *>(offset + (size_t)g * N + n0));
    const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w}, ow[4] = {oraw.x, oraw.y, oraw.z, oraw.w};
    float sc[8], of[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t sb = (i & 1) ? sw[i >> 1] >> 16 : sw[i >> 1] & 0xFFFFu, ob = (i & 1) ? ow[i >> 1] >> 16 : ow[i >> 1] & 0xFFFFu;
        if constexpr (BF16) { sc[i] = __uint_as_float(sb << 16); of[i] = __uint_as_float(ob << 16); }
        else { sc[i] = __half2float(__ushort_as_half((unsigned short)sb)); of[i] = __half2float(__ushort_as_half((unsigned short)ob)); }
    }
    // all loads of the thread first, then the conversions and stores
    uint2 raw[RPT];
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr) {
        const int k = k0 + wid + 8 * rr;
        raw[rr] = make_uint2(0u, 0u);
        if (k < K) {
            if constexpr (Q4) raw[rr].x = __ldg(reinterpret_cast<const uint32_t *>(w + ((size_t)k * N + n0) / 2));
            else raw[rr] = __ldg(reinterpret_cast<const uint2 *>(w + (size_t)k * N + n0));
        }
    }
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr) {
        const int k = k0 + wid + 8 * rr;
        if (k >= K) break;
        float v[8];
        if constexpr (Q4) {
            const uint32_t word = raw[rr].x;
#pragma unroll
            for (int i = 0; i < 8; ++i)   // two's-complement nibble -> q + 8 in the mantissa of 2^23
                v[i] = __uint_as_float(0x4B000000u | (((word >> (4 * i)) & 0xFu) ^ 8u)) - 8388616.f;
        } else {
            const uint32_t words[2] = {raw[rr].x, raw[rr].y};
#pragma unroll
            for (int i = 0; i < 8; ++i)
                v[i] = __uint_as_float(0x4B000000u | (((words[i >> 2] >> (8 * (i & 3))) & 0xFFu) ^ 0x80u)) - 8388736.f;
        }
        uint4 o;
        uint32_t *op = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) op[i] = pack2<OUT_BF16>((v[2 * i] - of[2 * i]) * sc[2 * i], (v[2 * i + 1] - of[2 * i + 1]) * sc[2 * i + 1]);
        *reinterpret_cast<uint4 *>(out + (size_t)k * N + n0) = o;
    }
}

// bf16 activations -> fp16 with one power-of-two scale per row: xh[m][k] = half(x[m][k] * 2^-e_m),
// rowscale[m] = 2^e_m, e_m chosen so that the row's largest magnitude lands in [2^14, 2^15).  A bf16
// value has 8 significant bits and fp16 holds 11, so the conversion is exact for every element within
// 2^-29 of the row's maximum (smaller ones fall into fp16's subnormals and lose low bits; their share
// of any dot product is below fp32 resolution).  Lets a bf16 problem run on the fp16 tensor-core path,
// where the dequantised weights keep 11 significant bits instead of bf16's 8.  One CTA per row.
__global__ void __launch_bounds__(256) rows_bf16_to_scaled_f16_kernel(const uint16_t *x, uint16_t *xh, float *rowscale, int K) {
    const size_t row = blockIdx.x;
    const uint16_t *xr = x + row * K;
    uint16_t *hr = xh + row * K;
    __shared__ float red[8];
    float amax = 0.f;
    // K % 8 == 0 and 16-byte aligned rows on this path
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(xr + k));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            amax = fmaxf(amax, fabsf(__uint_as_float(w[i] << 16)));
            amax = fmaxf(amax, fabsf(__uint_as_float(w[i] & 0xFFFF0000u)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    // fmaxf drops NaNs; an infinite or zero row keeps scale 1 (inf and NaN convert to themselves)
    int e = 0;
    if (amax > 0.f && amax < __int_as_float(0x7f800000)) {
        e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127 - 14;
        e = e < -100 ? -100 : e;
    }
    const float down = __uint_as_float((uint32_t)(127 - e) << 23), up = __uint_as_float((uint32_t)(127 + e) << 23);
    if (threadIdx.x == 0) rowscale[row] = up;
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(xr + k));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint4 o;
        uint32_t *op = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) op[i] = pack2<false>(__uint_as_float(w[i] << 16) * down, __uint_as_float(w[i] & 0xFFFF0000u) * down);
        *reinterpret_cast<uint4 *>(hr + k) = o;
    }
}

// MX operand [rows][cols] -> bf16.  along_cols: one scale per (row, col / 32) (operand A, [M][K]);
// otherwise one per (row / 32, col) (operand B, [K][N]).  One thread expands 16 consecutive columns.
__global__ void expand_mx_kernel(const uint8_t *src, int elem_type, const uint8_t *scales, int along_cols, uint16_t *out, int rows,
                                 int cols) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = cols / 16;
    if (t >= (int64_t)rows * per_row) return;
    const int r = (int)(t / per_row), c0 = (int)(t % per_row) * 16;
    float v[16];
    if (elem_type == ET_E2M1) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(src + ((size_t)r * cols + c0) / 2));
        const uint32_t words[2] = {raw.x, raw.y};
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = e2m1_to_float((words[i >> 3] >> (4 * (i & 7))) & 0xF);
    } else {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(src + (size_t)r * cols + c0));
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint8_t b = (uint8_t)((words[i >> 2] >> (8 * (i & 3))) & 0xFF);
            v[i] = elem_type == ET_E4M3 ? e4m3_to_float(b) : e5m2_to_float(b);
        }
    }
    if (along_cols) {
        const float s = e8m0_to_float(scales[(size_t)r * (cols / 32) + c0 / 32]);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] *= s;
    } else {
        const uint4 sraw = __ldg(reinterpret_cast<const uint4 *>(scales + (size_t)(r / 32) * cols + c0));
        const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] *= e8m0_to_float((sw[i >> 2] >> (8 * (i & 3))) & 0xFF);
    }
    uint4 o0, o1;
    o0.x = pack2<true>(v[0], v[1]);   o0.y = pack2<true>(v[2], v[3]);   o0.z = pack2<true>(v[4], v[5]);   o0.w = pack2<true>(v[6], v[7]);
    o1.x = pack2<true>(v[8], v[9]);   o1.y = pack2<true>(v[10], v[11]); o1.z = pack2<true>(v[12], v[13]); o1.w = pack2<true>(v[14], v[15]);
    uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)r * cols + c0);
    dst[0] = o0;
    dst[1] = o1;
}

// The same written for bandwidth, like expand_wq_fast_kernel: a lane owns 8 consecutive columns and
// walks 4 rows of a 32-row chunk; operand B loads its 8 scale bytes once per chunk, operand A one
// scale byte per row; one 16-byte store per row.  ELEM: 0 = e2m1 (two per byte), 1 = e4m3, 2 = e5m2.
template <int ELEM, bool ALONG_COLS>
__global__ void __launch_bounds__(256) expand_mx_fast_kernel(const uint8_t *src, const uint8_t *scales, uint16_t *out, int rows,
                                                             int cols) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int c0 = (blockIdx.x * 32 + lane) * 8;
    const int r0 = blockIdx.y * 32;
    if (c0 >= cols) return;
    float sc[8];
    if constexpr (!ALONG_COLS) {
        const uint2 sraw = __ldg(reinterpret_cast<const uint2 *>(scales + (size_t)(r0 / 32) * cols + c0));
        const uint32_t sw[2] = {sraw.x, sraw.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) sc[i] = e8m0_to_float((sw[i >> 2] >> (8 * (i & 3))) & 0xFFu);
    }
    // all loads of the thread first (the stores below would otherwise order them), then the conversions
    uint2 rawv[4];
    uint32_t srow[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        const int r = r0 + wid + 8 * rr;
        rawv[rr] = make_uint2(0u, 0u);
        srow[rr] = 127u;
        if (r < rows) {
            if constexpr (ELEM == 0) rawv[rr].x = __ldg(reinterpret_cast<const uint32_t *>(src + ((size_t)r * cols + c0) / 2));
            else rawv[rr] = __ldg(reinterpret_cast<const uint2 *>(src + (size_t)r * cols + c0));
            if constexpr (ALONG_COLS) srow[rr] = __ldg(scales + (size_t)r * (cols / 32) + c0 / 32);
        }
    }
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        const int r = r0 + wid + 8 * rr;
        if (r >= rows) break;
        float v[8];
        if constexpr (ELEM == 0) {
            const uint32_t word = rawv[rr].x;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = e2m1_to_float((word >> (4 * i)) & 0xFu);
        } else {
            const uint2 raw = rawv[rr];
            const uint32_t words[2] = {raw.x, raw.y};
#pragma unroll
            for (int i = 0; i < 4; ++i) {   // two fp8 at a time through the hardware conversion
                const __nv_fp8x2_storage_t pair = (__nv_fp8x2_storage_t)((words[i >> 1] >> (16 * (i & 1))) & 0xFFFFu);
                const __half2 h2 = __half2(__nv_cvt_fp8x2_to_halfraw2(pair, ELEM == 1 ? __NV_E4M3 : __NV_E5M2));
                const float2 f2 = __half22float2(h2);
                v[2 * i] = f2.x;
                v[2 * i + 1] = f2.y;
            }
        }
        if constexpr (ALONG_COLS) {
            const float s1 = e8m0_to_float(srow[rr]);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= s1;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= sc[i];
        }
        uint4 o;
        uint32_t *op = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) op[i] = pack2<true>(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(out + (size_t)r * cols + c0) = o;
    }
}

template <bool ALONG_COLS>
bool launch_expand_mx_fast(const uint8_t *src, int elem_type, const uint8_t *scales, uint16_t *out, int rows, int cols, cudaStream_t s) {
    if (cols % 32 != 0 || (reinterpret_cast<uintptr_t>(src) & 7) || (reinterpret_cast<uintptr_t>(scales) & 7) || (rows + 31) / 32 > 65535)
        return false;
    if (!ALONG_COLS && rows % 32 != 0) return false;
    const dim3 grid((unsigned)((cols + 255) / 256), (unsigned)((rows + 31) / 32));
    if (elem_type == ET_E2M1) expand_mx_fast_kernel<0, ALONG_COLS><<<grid, 256, 0, s>>>(src, scales, out, rows, cols);
    else if (elem_type == ET_E4M3) expand_mx_fast_kernel<1, ALONG_COLS><<<grid, 256, 0, s>>>(src, scales, out, rows, cols);
    else if (elem_type == ET_E5M2) expand_mx_fast_kernel<2, ALONG_COLS><<<grid, 256, 0, s>>>(src, scales, out, rows, cols);
    else return false;
    return true;
}

inline uint64_t up256(uint64_t x) { return (x + 255) / 256 * 256; }
bool is_mx(const MatmulArgs &p) { return p.a_scale && p.b_scale; }

// Weight-only matmuls with bf16 activations run their tensor-core product in fp16: the activations are
// converted with a power-of-two scale per row (exact, see rows_bf16_to_scaled_f16_kernel), the weights
// are expanded to fp16 -- (q - offset) * scale of a 4- or 8-bit integer and a bf16 scale then keeps 11
// significant bits (exact without an offset for int4) instead of being rounded to bf16's 8 -- and the
// epilogue multiplies the row scale back in fp32.  Against the exact product the mean error of the
// bf16 output drops from 2.1e-3 (bf16 weights) to 1.4e-3 (its own rounding alone).
// B200_QMM_WQ_BF16_VIA_F16=0 keeps bf16 weights.
bool via_f16(const MatmulArgs &p) {
    if (is_mx(p) || p.a_type != ET_BF16) return false;
    const char *e = getenv("B200_QMM_WQ_BF16_VIA_F16");
    return !(e && atoi(e) == 0);
}

// The dense problem that remains once the operands are expanded.
MatmulArgs dense_args(const MatmulArgs &p, void *a16, void *b16, const float *rowscale = nullptr) {
    MatmulArgs d;
    d.a = a16; d.b = b16; d.out = p.out;
    d.a_type = d.b_type = is_mx(p) ? (int)ET_BF16 : (via_f16(p) ? (int)ET_F16 : p.a_type);
    d.out_type = p.out_type;
    d.bias = p.bias; d.bias_type = p.bias_type;
    d.pertoken = rowscale;
    d.epilogue = EPI_PLAIN;
    d.M = p.M; d.N = p.N; d.K = p.K; d.group = p.K;
    return d;
}

struct ExpandLayout { uint64_t a_bytes, rs_bytes, b_bytes; };
ExpandLayout expand_layout(const MatmulArgs &p) {
    ExpandLayout l{};
    const bool a_copy = is_mx(p) || via_f16(p);
    l.a_bytes = a_copy ? up256((uint64_t)p.M * p.K * 2) : 0;
    l.rs_bytes = via_f16(p) ? up256((uint64_t)p.M * sizeof(float)) : 0;
    l.b_bytes = up256((uint64_t)p.K * p.N * 2);
    return l;
}

}  // namespace

bool expand_supported(const MatmulArgs &p) {
    if (p.epilogue != EPI_PLAIN || p.batch != 1 || p.b_transposed || p.accumulate || p.M < 1) return false;
    if (p.K % 32 != 0 || p.N % 16 != 0) return false;
    if (is_mx(p)) {
        auto ok = [](int t) { return t == ET_E4M3 || t == ET_E5M2 || t == ET_E2M1; };
        if (!ok(p.a_type) || !ok(p.b_type)) return false;
    } else {
        if (!p.scale) return false;
        if (p.a_type != ET_F16 && p.a_type != ET_BF16) return false;
        if (p.b_type != ET_I4 && p.b_type != ET_I8) return false;
        if (p.sc_type != p.a_type || p.out_type != p.a_type || (p.bias && p.bias_type != p.a_type)) return false;
        if (p.group < p.K && p.K % p.group != 0) return false;
    }
    return dense_tc_supported(dense_args(p, nullptr, nullptr));
}

uint64_t expand_workspace_bytes(const MatmulArgs &p) {
    const ExpandLayout l = expand_layout(p);
    return l.a_bytes + l.rs_bytes + l.b_bytes + dense_tc_workspace_bytes(dense_args(p, nullptr, nullptr));
}

cudaError_t launch_expand(const MatmulArgs &p, cudaStream_t s) {
    if (!p.workspace || p.workspace_bytes < expand_workspace_bytes(p)) return cudaErrorInvalidValue;
    // refused before anything is launched: operands and output off the 16-byte alignment of the dense kernel
    auto misaligned16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
    if (misaligned16(p.a) || misaligned16(p.b) || misaligned16(p.out) || misaligned16(p.workspace) ||
        (is_mx(p) && misaligned16(p.b_scale)))
        return cudaErrorMisalignedAddress;
    char *ws = (char *)p.workspace;
    const ExpandLayout l = expand_layout(p);
    const uint64_t a_bytes = l.a_bytes + l.rs_bytes, b_bytes = l.b_bytes;
    uint16_t *a16 = (uint16_t *)ws, *b16 = (uint16_t *)(ws + a_bytes);
    float *rowscale = l.rs_bytes ? (float *)(ws + l.a_bytes) : nullptr;
    const bool f16w = via_f16(p);   // weights expanded to fp16 under bf16 scales
    const int K = (int)p.K, N = (int)p.N, M = (int)p.M;
    if (is_mx(p)) {
        const int64_t ta = (int64_t)M * (K / 16), tb = (int64_t)K * (N / 16);
        if (!launch_expand_mx_fast<true>((const uint8_t *)p.a, p.a_type, (const uint8_t *)p.a_scale, a16, M, K, s))
            expand_mx_kernel<<<(unsigned)((ta + 255) / 256), 256, 0, s>>>((const uint8_t *)p.a, p.a_type, p.a_scale, 1, a16, M, K);
        count_launch();
        if (!launch_expand_mx_fast<false>((const uint8_t *)p.b, p.b_type, (const uint8_t *)p.b_scale, b16, K, N, s))
            expand_mx_kernel<<<(unsigned)((tb + 255) / 256), 256, 0, s>>>((const uint8_t *)p.b, p.b_type, p.b_scale, 0, b16, K, N);
        count_launch();
    } else {
        const int64_t tb = (int64_t)K * (N / 16);
        const unsigned blocks = (unsigned)((tb + 255) / 256);
        const bool q4 = p.b_type == ET_I4, bf = p.a_type == ET_BF16;
        const uint8_t *w = (const uint8_t *)p.b;
        const bool fast = p.sc_type == p.a_type && N % 8 == 0 && (p.group >= p.K || p.group % 32 == 0) &&
                          (reinterpret_cast<uintptr_t>(p.scale) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.offset) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(p.b) & 7) == 0 && (K + 31) / 32 <= 65535;
        if (f16w) {
            rows_bf16_to_scaled_f16_kernel<<<(unsigned)M, 256, 0, s>>>((const uint16_t *)p.a, a16, rowscale, K);
            count_launch();
        }
        if (fast) {
            const uint16_t *sc16 = (const uint16_t *)p.scale, *of16 = (const uint16_t *)p.offset;
            // 8 rows per thread (64-row blocks) where a block still sits inside one scale group
            // (measured on 8192 x 28672 at M = 512: 287 us with 4 rows per thread, 276 with 8, 280 with 16)
            const int rpt = (p.group >= p.K || p.group % 64 == 0) ? 8 : 4;
            const int rows = 8 * rpt;
            const dim3 grid((unsigned)((N + 255) / 256), (unsigned)((K + rows - 1) / rows));
            const int grp = p.group >= p.K ? (K + rows - 1) / rows * rows : (int)p.group;   // per-channel: one group over all rows
#define EXPAND_WQ(Q, B, OB) do { if (rpt == 8) expand_wq_fast_kernel<Q, B, 8, OB><<<grid, 256, 0, s>>>(w, sc16, of16, b16, K, N, grp); \
                                 else expand_wq_fast_kernel<Q, B, 4, OB><<<grid, 256, 0, s>>>(w, sc16, of16, b16, K, N, grp); } while (0)
            if (q4 && bf && f16w) EXPAND_WQ(true, true, false);
            else if (bf && f16w) EXPAND_WQ(false, true, false);
            else if (q4 && bf) EXPAND_WQ(true, true, true);
            else if (q4) EXPAND_WQ(true, false, false);
            else if (bf) EXPAND_WQ(false, true, true);
            else EXPAND_WQ(false, false, false);
#undef EXPAND_WQ
        } else if (q4 && bf && f16w) expand_wq_kernel<true, true, false><<<blocks, 256, 0, s>>>(w, p.scale, p.offset, p.sc_type, b16, K, N, (int)p.group);
        else if (bf && f16w) expand_wq_kernel<false, true, false><<<blocks, 256, 0, s>>>(w, p.scale, p.offset, p.sc_type, b16, K, N, (int)p.group);
        else if (q4 && bf) expand_wq_kernel<true, true><<<blocks, 256, 0, s>>>(w, p.scale, p.offset, p.sc_type, b16, K, N, (int)p.group);
        else if (q4) expand_wq_kernel<true, false><<<blocks, 256, 0, s>>>(w, p.scale, p.offset, p.sc_type, b16, K, N, (int)p.group);
        else if (bf) expand_wq_kernel<false, true><<<blocks, 256, 0, s>>>(w, p.scale, p.offset, p.sc_type, b16, K, N, (int)p.group);
        else expand_wq_kernel<false, false><<<blocks, 256, 0, s>>>(w, p.scale, p.offset, p.sc_type, b16, K, N, (int)p.group);
        count_launch();
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    MatmulArgs d = dense_args(p, (is_mx(p) || f16w) ? (void *)a16 : const_cast<void *>(p.a), b16, rowscale);
    d.workspace = ws + a_bytes + b_bytes;
    d.workspace_bytes = p.workspace_bytes - a_bytes - b_bytes;
    return launch_dense_tc(d, s);
}

cudaError_t launch_rows_bf16_to_scaled_f16(const void *x, void *xh, float *rowscale, int64_t M, int64_t K, cudaStream_t s) {
    if (M <= 0 || K <= 0 || (K & 7)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(xh) & 15)) return cudaErrorMisalignedAddress;
    rows_bf16_to_scaled_f16_kernel<<<(unsigned)M, 256, 0, s>>>((const uint16_t *)x, (uint16_t *)xh, rowscale, (int)K);
    count_launch();
    return cudaGetLastError();
}

}  // namespace qmm
