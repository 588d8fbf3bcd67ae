// HBM-bound streaming kernel for weight-only quantized matmul at very small M (decode).
//
// Replaces the reference's k_wq_fused (cuda/src/ops/matmul.cu:337-352: one thread per output
// column, serial K loop, scalar 1-byte loads, at most N/256 CTAs).  Here:
//   * every thread streams 16-byte (or 8-byte) vectors of packed int4 / int8 weights along N,
//   * lanes of a warp are split LN along N x LK along K, warps of a CTA and CTAs of the grid split K
//     further (split-K), so any N fills all 148 SMs,
//   * weights are converted in registers (byte-permute + magic-number float), activations sit in
//     shared memory as fp32, accumulation is fp32,
//   * the antiquant algebra is the reference's: sum_k a*(q-off)*s = s*(sum a*q - off*sum a)
//     (matmul.cu:334-335), applied once per scale group by the warp that owns the group,
//   * partial sums are reduced with warp shuffles (across LK), shared memory (across warps) and,
//     when split_k > 1, fp32 partials in the caller's workspace that a second kernel reduces.
#include "device_utils.cuh"

namespace qmm {
namespace {

constexpr int MAX_SLICE_ROWS = 2048;  // activation rows of K staged per CTA (fp32, per m)

struct GemvParams {
    const void *x;
    const uint8_t *w;
    const void *scale;
    const void *offset;
    const void *bias;
    void *out;
    float *partial;  // [split_k][M][N] fp32, or null when split_k == 1
    int M, N, K;
    int vg;          // rows per scale group (or per virtual group for per-channel scales)
    int grouped;     // 1: scale/offset are [K/vg, N]; 0: [N]
    int slice;       // rows of K per CTA (multiple of vg)
    int x_type, out_type;
};

template <int WBITS, int VB>
struct WeightVec {
    static constexpr int C = VB * 8 / WBITS;  // columns per thread
    uint32_t r[VB / 4];
    __device__ __forceinline__ void load(const uint8_t *p) {
        if constexpr (VB == 16) {
            uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
            r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
        } else {
            uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
            r[0] = v.x; r[1] = v.y;
        }
    }
    // Column j as float.  int8: byte j; int4: nibble j (low nibble first).
    __device__ __forceinline__ void decode(float (&f)[C]) const {
        if constexpr (WBITS == 8) {
#pragma unroll
            for (int i = 0; i < VB / 4; ++i) {
                uint32_t u = r[i] ^ 0x80808080u;  // two's complement -> offset binary (v + 128)
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    f[i * 4 + b] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540 | b)) - 8388736.f;  // 2^23 + 128
            }
        } else {
#pragma unroll
            for (int i = 0; i < VB / 4; ++i) {
                uint32_t u = r[i] ^ 0x88888888u;  // v + 8 in every nibble
                uint32_t lo = u & 0x0F0F0F0Fu, hi = (u >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    f[i * 8 + 2 * b] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7540 | b)) - 8388616.f;  // 2^23 + 8
                    f[i * 8 + 2 * b + 1] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7540 | b)) - 8388616.f;
                }
            }
        }
    }
};

template <int WBITS, int MT, int VB, int LN, int NWARP>
__global__ void __launch_bounds__(NWARP * 32) gemv_kernel(const GemvParams p) {
    using Vec = WeightVec<WBITS, VB>;
    constexpr int C = Vec::C, LK = 32 / LN, TN = LN * C;
    extern __shared__ float smem[];
    float *xs = smem;                         // [MT][slice]
    float *red = smem + MT * MAX_SLICE_ROWS;  // [NWARP][MT][TN]

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, ln = lane % LN, lk = lane / LN;
    const int n_base = blockIdx.x * TN + ln * C;
    const int kb = blockIdx.y * p.slice, ke = min(p.K, kb + p.slice);
    const bool col_ok = n_base < p.N;  // N is a multiple of C, so a thread's columns are all in or all out

    for (int i = threadIdx.x; i < MT * (ke - kb); i += NWARP * 32) {
        int m = i / (ke - kb), k = i % (ke - kb);
        xs[m * MAX_SLICE_ROWS + k] = m < p.M ? load_as_float(p.x, p.x_type, (int64_t)m * p.K + kb + k) : 0.f;
    }
    __syncthreads();

    float tot[MT][C];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < C; ++j) tot[m][j] = 0.f;

    if (col_ok) {
        float acc[MT][C], sa[MT];
        const size_t row_bytes = (size_t)p.N * WBITS / 8;
        const uint8_t *wcol = p.w + (size_t)n_base * WBITS / 8;
        auto clear = [&]() {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                sa[m] = 0.f;
#pragma unroll
                for (int j = 0; j < C; ++j) acc[m][j] = 0.f;
            }
        };
        // tot += s * (acc - off * sa) with this group's (or the per-channel) scale row.
        auto fold = [&](int g) {
            const size_t srow = (size_t)g * p.N + n_base;
#pragma unroll
            for (int j = 0; j < C; ++j) {
                float s = load_as_float(p.scale, p.x_type, srow + j);
                float o = p.offset ? load_as_float(p.offset, p.x_type, srow + j) : 0.f;
#pragma unroll
                for (int m = 0; m < MT; ++m) tot[m][j] = fmaf(s, acc[m][j] - o * sa[m], tot[m][j]);
            }
        };
        clear();
        for (int g0 = kb + warp * p.vg; g0 < ke; g0 += NWARP * p.vg) {
            const int rows = min(p.vg, ke - g0);
            for (int r0 = lk; r0 < rows; r0 += 4 * LK) {
                Vec v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (r0 + u * LK < rows) v[u].load(wcol + (size_t)(g0 + r0 + u * LK) * row_bytes);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (r0 + u * LK >= rows) break;
                    float f[C];
                    v[u].decode(f);
                    const int kx = g0 + r0 + u * LK - kb;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float a = xs[m * MAX_SLICE_ROWS + kx];
                        sa[m] += a;
#pragma unroll
                        for (int j = 0; j < C; ++j) acc[m][j] = fmaf(a, f[j], acc[m][j]);
                    }
                }
            }
            if (p.grouped) { fold(g0 / p.vg); clear(); }
        }
        if (!p.grouped) fold(0);
    }

    // Across the LK lanes that share columns, then across warps.
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < C; ++j) {
            float v = tot[m][j];
#pragma unroll
            for (int d = LN; d < 32; d <<= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            tot[m][j] = v;
        }
    if (lk == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < C; ++j) red[(warp * MT + m) * TN + ln * C + j] = tot[m][j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < MT * TN; i += NWARP * 32) {
        int m = i / TN, c = i % TN, n = blockIdx.x * TN + c;
        if (m >= p.M || n >= p.N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) v += red[(w * MT + m) * TN + c];
        if (p.partial) {
            p.partial[((size_t)blockIdx.y * p.M + m) * p.N + n] = v;
        } else {
            if (p.bias) v += load_as_float(p.bias, p.x_type, n);
            store_from_float(p.out, p.out_type, (int64_t)m * p.N + n, v);
        }
    }
}

// out[m,n] = T(sum_s partial[s][m][n] + bias[n])
__global__ void gemv_finalize_kernel(const float *partial, const void *bias, void *out, int M, int N, int split_k,
                                     int x_type, int out_type) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)M * N) return;
    float v = 0.f;
    for (int s = 0; s < split_k; ++s) v += partial[(size_t)s * M * N + i];
    if (bias) v += load_as_float(bias, x_type, i % N);
    store_from_float(out, out_type, i, v);
}

template <int WBITS, int MT, int VB, int LN, int NWARP>
cudaError_t run(const GemvParams &gp, int split_k, cudaStream_t s) {
    constexpr int TN = LN * (VB * 8 / WBITS);
    size_t smem = (size_t)(MT * MAX_SLICE_ROWS + NWARP * MT * TN) * sizeof(float);
    auto kern = gemv_kernel<WBITS, MT, VB, LN, NWARP>;
    static bool attr_set[64] = {};  // per device; a racing second call sets the same value
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    dim3 grid((gp.N + TN - 1) / TN, split_k);
    kern<<<grid, NWARP * 32, smem, s>>>(gp);
    count_launch();
    return cudaGetLastError();
}

int virtual_group(const MatmulArgs &p) {
    if (p.group < p.K) return (int)p.group;
    for (int vg : {128, 64, 32, 16, 8}) if (p.K % vg == 0) return vg;
    return 0;
}

}  // namespace

int gemv_max_m() { return 4; }

bool gemv_supported(const MatmulArgs &p) {
    if (p.epilogue != EPI_PLAIN || p.batch != 1 || p.b_transposed || p.accumulate) return false;
    if (p.M < 1 || p.M > gemv_max_m()) return false;
    if (p.b_type != ET_I8 && p.b_type != ET_I4) return false;
    if (p.a_type != ET_F16 && p.a_type != ET_BF16 && p.a_type != ET_F32) return false;
    if (p.sc_type != p.a_type || (p.bias && p.bias_type != p.a_type)) return false;
    if (p.N % 32 != 0) return false;  // 16-byte vectors of int4 along N
    int vg = virtual_group(p);
    if (vg == 0 || p.K % vg != 0 || vg % 8 != 0 || vg > MAX_SLICE_ROWS) return false;
    if (p.K > (1 << 24) || p.N > (1 << 24)) return false;
    return true;
}

int gemv_pick_split_k(const MatmulArgs &p) {
    const int vg = virtual_group(p);
    const int groups = (int)(p.K / vg);
    const int tn = 256;  // widest CTA tile below (LN=8, 32 columns per thread)
    const int n_tiles = (int)((p.N + tn - 1) / tn);
    // Aim for ~4 CTAs per SM; every CTA needs at least one group per warp-pass and at most
    // MAX_SLICE_ROWS rows.
    int want = (4 * 148 + n_tiles - 1) / n_tiles;
    int min_split = (int)((p.K + MAX_SLICE_ROWS - 1) / MAX_SLICE_ROWS);
    int split = want < min_split ? min_split : want;
    if (split > groups) split = groups;
    // slices are whole groups
    int gps = (groups + split - 1) / split;
    while ((int64_t)gps * vg > MAX_SLICE_ROWS) --gps;
    return (groups + gps - 1) / gps;
}

uint64_t gemv_workspace_bytes(const MatmulArgs &p) {
    return p.split_k > 1 ? (uint64_t)p.split_k * p.M * p.N * sizeof(float) : 0;
}

cudaError_t launch_gemv(const MatmulArgs &p, cudaStream_t s) {
    GemvParams gp;
    gp.x = p.a; gp.w = (const uint8_t *)p.b; gp.scale = p.scale; gp.offset = p.offset; gp.bias = p.bias; gp.out = p.out;
    gp.M = (int)p.M; gp.N = (int)p.N; gp.K = (int)p.K;
    gp.vg = virtual_group(p);
    gp.grouped = p.group < p.K ? 1 : 0;
    const int groups = gp.K / gp.vg;
    const int split = p.split_k < 1 ? 1 : p.split_k;
    const int gps = (groups + split - 1) / split;
    gp.slice = gps * gp.vg;
    gp.x_type = p.a_type; gp.out_type = p.out_type;
    gp.partial = split > 1 ? (float *)p.workspace : nullptr;
    if (split > 1 && p.workspace_bytes < gemv_workspace_bytes(p)) return cudaErrorInvalidValue;
    if (gp.slice > MAX_SLICE_ROWS) return cudaErrorInvalidValue;
    // The kernel reads the packed weights with 16-byte loads (8-byte ones for 3..4 rows): a weight
    // pointer off that boundary would fault on the device, so it is refused here instead.
    if (reinterpret_cast<uintptr_t>(p.b) & (p.M <= 2 ? 15 : 7)) return cudaErrorMisalignedAddress;

    cudaError_t e;
    const bool w4 = p.b_type == ET_I4;
    if (p.M == 1)      e = w4 ? run<4, 1, 16, 8, 4>(gp, split, s) : run<8, 1, 16, 8, 4>(gp, split, s);
    else if (p.M == 2) e = w4 ? run<4, 2, 16, 8, 4>(gp, split, s) : run<8, 2, 16, 8, 4>(gp, split, s);
    else               e = w4 ? run<4, 4, 8, 8, 4>(gp, split, s) : run<8, 4, 8, 8, 4>(gp, split, s);
    if (e != cudaSuccess) return e;
    if (split > 1) {
        int64_t mn = p.M * p.N;
        gemv_finalize_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(gp.partial, p.bias, p.out, gp.M, gp.N, split,
                                                                           p.a_type, p.out_type);
        count_launch();
        e = cudaGetLastError();
    }
    return e;
}

// ---------------------------------------------------------------------------------------------
// Decode matmul for callers that cannot hand over scratch memory.
//
// The split-K partial sums of the streaming kernel normally live in the caller's workspace.  Some
// programs written against the reference have no workspace to give on this path: the reference
// reports 0 workspace bytes for M <= 16 (cuda/src/ops/matmul.cu:773-774), so their decode loop was
// built without one, and it runs at a point where device memory can no longer be requested (the
// device arena was carved up at start-up and allocation calls are forbidden in the serving loop).
// For them the partial sums go into the fixed array below, which every GPU that loads this library
// holds until the process exits.
//
// The array is shared by all calls and keeps the previous call's contents.  The kernels overwrite
// every element they later read, so nothing has to be cleared; two calls whose kernels overlap on
// the GPU (different streams, different threads) would race on it and must be serialised by the
// caller.
constexpr size_t NOALLOC_SCRATCH_FLOATS = 512 * 1024;  // 2 MiB per GPU
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

size_t noalloc_scratch_bytes() { return NOALLOC_SCRATCH_FLOATS * sizeof(float); }

// Device address of the scratch array on the current device.  In host code the array's name is
// only a handle for the runtime, not a device pointer, so the address is looked up once per device
// (with that device current) and cached.
static cudaError_t noalloc_scratch_ptr(float **out) {
    // Filled without a lock: two threads making the first call on a device may both look the address
    // up; they store the same value, so the race is harmless.
    static float *cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!cached[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return cudaSuccess;
}

cudaError_t launch_gemv_noalloc(MatmulArgs p, cudaStream_t s, bool *too_large) {
    *too_large = false;
    p.split_k = gemv_pick_split_k(p);
    const uint64_t need = gemv_workspace_bytes(p);
    if (need > noalloc_scratch_bytes()) {
        *too_large = true;
        return cudaErrorInvalidValue;
    }
    float *scratch = nullptr;
    cudaError_t e = noalloc_scratch_ptr(&scratch);
    if (e != cudaSuccess) return e;
    p.workspace = scratch;
    p.workspace_bytes = noalloc_scratch_bytes();
    return launch_gemv(p, s);
}

}  // namespace qmm
