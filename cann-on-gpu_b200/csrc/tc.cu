// tcgen05 tensor-core kernels of the quantized-matmul family (sm_100a only).
//
// One warp-specialised kernel template covers W8A8 and the weight-only (W4A16 / W8A16) matmuls:
//
//   * The WEIGHT tile sits on the MMA's M side (128 output columns n per CTA) and the ACTIVATION tile
//     on its N side (MT = 16..256 rows m).  The caller's weight is [K,N] with N contiguous, which is
//     exactly the "MN-major" operand form of tcgen05.mma for 8- and 16-bit types, so no transpose pass
//     exists anywhere (the reference transposes the whole weight on every call,
//     cuda/src/ops/matmul.cu:824).  Small M costs nothing: the instruction's N extent shrinks to 16.
//   * Accumulators live in TMEM: lane = output column n, TMEM column = output row m.  Everything that
//     is indexed by n (scale, offset, bias) is therefore a per-thread scalar in the epilogue.
//   * W8A8: int8 weights and activations go from HBM to swizzled shared memory by TMA and straight
//     into kind::i8 MMAs; the int32 accumulators are exact; the epilogue applies
//     float(acc + bias) * scale[n] * pertoken[m] and the output cast (the reference runs an int8
//     GEMM into a workspace and a separate scale kernel, matmul.cu:825-846).
//   * W4A16 / W8A16: TMA stages the PACKED weights; four converter warps expand them in registers to
//     bf16/fp16 INTEGERS (exact) and write them in the MMA's canonical swizzled layout; kind::f16 MMAs
//     accumulate sum_k x*q per scale group in TMEM, and the epilogue warps fold every finished group
//     into fp32 registers with the reference's algebra s*(sum x*q - off*sum x) (matmul.cu:334-335).
//     Weights are never rounded and no dequantised copy is ever written (the reference materialises
//     K*N fp16 weights per call for M > 16, matmul.cu:790-795).
//   * Warp roles: 0 = TMA producer, 1 = MMA issuer (+TMEM owner), 2..5 = epilogue, 6..9 = converters.
//     Stages are handed over with mbarriers; tcgen05.commit signals stage release and accumulator
//     completion.  Two TMEM accumulators alternate between scale groups so the fold of group g
//     overlaps the MMAs of group g+1.
//   * Split-K over gridDim.z fills the 148 SMs at decode shapes; partial sums go to the caller's
//     workspace and a small second kernel reduces them and applies bias / dequant / cast.
//   * Every wait is bounded: after about a second a thread records a code in a status word, raises
//     a CTA-wide abort flag and all roles fall through to the common exit, which frees the TMEM.
#include <cstring>
#include <mutex>

#include "tc_common.cuh"

namespace qmm {
namespace {

enum WMode : int {
    W_I8 = 0,    // int8 weights by TMA straight into kind::i8
    W_Q4_BF16,   // packed int4 -> bf16 integers, kind::f16
    W_Q4_F16,    // packed int4 -> fp16 integers
    W_Q8_BF16,   // int8 -> bf16 integers
    W_Q8_F16,    // int8 -> fp16 integers
};

template <int WMODE> struct WTraits;
template <> struct WTraits<W_I8>      { static constexpr int BK = 128, STAGE_W = 0,    UMMA_K = 32, W_KSTEP = 4096, W_LBO = 16384; static constexpr bool CVT = false, Q4 = false, BF16 = false; };
template <> struct WTraits<W_Q4_BF16> { static constexpr int BK = 64,  STAGE_W = 4096, UMMA_K = 16, W_KSTEP = 2048, W_LBO = 8192;  static constexpr bool CVT = true,  Q4 = true,  BF16 = true; };
template <> struct WTraits<W_Q4_F16>  { static constexpr int BK = 64,  STAGE_W = 4096, UMMA_K = 16, W_KSTEP = 2048, W_LBO = 8192;  static constexpr bool CVT = true,  Q4 = true,  BF16 = false; };
template <> struct WTraits<W_Q8_BF16> { static constexpr int BK = 64,  STAGE_W = 8192, UMMA_K = 16, W_KSTEP = 2048, W_LBO = 8192;  static constexpr bool CVT = true,  Q4 = false, BF16 = true; };
template <> struct WTraits<W_Q8_F16>  { static constexpr int BK = 64,  STAGE_W = 8192, UMMA_K = 16, W_KSTEP = 2048, W_LBO = 8192;  static constexpr bool CVT = true,  Q4 = false, BF16 = false; };

constexpr int TILE_N = 128;          // output columns per CTA = MMA M
constexpr int W_TILE_BYTES = 16384;  // MMA-ready weight tile per stage (128 n x 128 B of K, or 2 x 64 k x 128 B)
constexpr int MAX_UNITS = 64;        // scale groups (fold units) per CTA

struct TcParams {
    void *out;
    void *partial;            // [split][M][N] fp32 or int32 raw accumulators, or null
    const void *scale;        // W8A8: [N]; weight-only: [G,N]
    const void *offset;       // weight-only: [G,N] or null
    const void *bias;
    const float *pertoken;
    const float *xsum;        // [units][M] sums of activations per fold unit (weight-only with offset)
    int sc_type, bias_type, out_type, epilogue;
    int M, N, K;
    int num_kb;               // K blocks in total
    int kb_per_split;         // K blocks per CTA along gridDim.z
    int kb_per_unit;          // K blocks per fold unit (scale group); kb_per_split for per-channel scales
    int grouped;              // scale rows per group (1) or one row for all of K (0)
};

// ------------------------------------------------------------------------------------------------ kernel
template <int WMODE, int MT, int STAGES>
struct SmemLayout {
    using T = WTraits<WMODE>;
    static constexpr int X_BYTES = MT * 128;
    static constexpr int STAGE_BYTES = X_BYTES + W_TILE_BYTES + T::STAGE_W;
    static constexpr int XS_FLOATS = T::CVT ? 4096 : 0;  // activation sums of this CTA's fold units
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 3 * STAGES + 4;
    static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
    static constexpr int XS_OFF = (MISC_OFF + 16 + 15) / 16 * 16;
    static constexpr int TOTAL = XS_OFF + XS_FLOATS * 4 + 1024;  // + slack for the 1024-byte base alignment
};

template <int WMODE, int MT, int STAGES>
__global__ void __launch_bounds__(WTraits<WMODE>::CVT ? 320 : 192, 1)
tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const TcParams p) {
    using T = WTraits<WMODE>;
    using L = SmemLayout<WMODE, MT, STAGES>;
    constexpr bool INT8 = (WMODE == W_I8);
    constexpr int NACC = MT <= 128 ? 2 : 1;
    constexpr int TMEM_COLS = (NACC * MT) < 32 ? 32 : (NACC * MT);  // powers of two by construction
    constexpr int KSTEPS = T::BK / T::UMMA_K;
    constexpr uint32_t IDESC = INT8 ? instr_desc(2, 1, TILE_N, MT) : instr_desc(1, T::BF16 ? 1 : 0, TILE_N, MT);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    auto x_tile = [&](int s) { return base + s * L::STAGE_BYTES; };
    auto w_tile = [&](int s) { return base + s * L::STAGE_BYTES + L::X_BYTES; };
    auto w_stage = [&](int s) { return base + s * L::STAGE_BYTES + L::X_BYTES + W_TILE_BYTES; };
    auto bar_full = [&](int s) { return base + L::BAR_OFF + 8 * s; };
    auto bar_empty = [&](int s) { return base + L::BAR_OFF + 8 * (STAGES + s); };
    auto bar_wready = [&](int s) { return base + L::BAR_OFF + 8 * (2 * STAGES + s); };
    auto bar_acc_full = [&](int a) { return base + L::BAR_OFF + 8 * (3 * STAGES + a); };
    auto bar_acc_empty = [&](int a) { return base + L::BAR_OFF + 8 * (3 * STAGES + 2 + a); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen_base + L::MISC_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + L::MISC_OFF + 4);
    float *xs_sm = reinterpret_cast<float *>(gen_base + L::XS_OFF);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TILE_N, m0 = blockIdx.y * MT;
    const int kb0 = blockIdx.z * p.kb_per_split;
    const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
    const int nkb = kb1 - kb0;                                   // > 0 by construction of the grid
    const int units = (nkb + p.kb_per_unit - 1) / p.kb_per_unit; // fold units of this CTA

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
            mbar_init(bar_wready(s), 4);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void *)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(bar_empty(s), ((i / STAGES) - 1) & 1, abort_flag, 1)) break;
                mbar_expect_tx(bar_full(s), L::X_BYTES + (T::CVT ? T::STAGE_W : W_TILE_BYTES));
                const int k = (kb0 + i) * T::BK;
                tma_load_2d(x_tile(s), &tm_x, bar_full(s), k, m0);
                if constexpr (T::CVT) tma_load_2d(w_stage(s), &tm_w, bar_full(s), T::Q4 ? n0 / 2 : n0, k);
                else tma_load_2d(w_tile(s), &tm_w, bar_full(s), n0, k);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES, u = i / p.kb_per_unit, a = u % NACC;
                const bool unit_start = (i % p.kb_per_unit) == 0;
                if (unit_start && u >= NACC && !mbar_wait(bar_acc_empty(a), ((u / NACC) - 1) & 1, abort_flag, 2)) break;
                if (!mbar_wait(bar_full(s), (i / STAGES) & 1, abort_flag, 3)) break;
                if constexpr (T::CVT) { if (!mbar_wait(bar_wready(s), (i / STAGES) & 1, abort_flag, 4)) break; }
                tc_fence_after();
                const uint32_t d = tmem_base + a * MT;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    const uint64_t a_desc = smem_desc(w_tile(s) + kk * T::W_KSTEP, T::W_LBO, 1024);
                    const uint64_t b_desc = smem_desc(x_tile(s) + kk * 32, 16, 1024);
                    tc_mma<INT8>(d, a_desc, b_desc, IDESC, (!unit_start || kk > 0) ? 1u : 0u);
                }
                tc_commit(bar_empty(s));
                if ((i + 1) % p.kb_per_unit == 0 || i + 1 == nkb) tc_commit(bar_acc_full(a));
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int r = q * 32 + lane;                  // accumulator lane
        const int n = n0 + col_of_lane<T::Q4>(r);
        const bool n_ok = n < p.N;
        const bool use_xs = T::CVT && p.offset != nullptr;
        if (use_xs) {
            // activation sums of this CTA's fold units: xs_sm[u][c] = xsum[unit0 + u][m0 + c]
            const int unit0 = kb0 / p.kb_per_unit;
            for (int i = threadIdx.x - 64; i < units * MT; i += 128) {
                const int u = i / MT, c = i % MT;
                xs_sm[i] = (m0 + c < p.M) ? p.xsum[(size_t)(unit0 + u) * p.M + m0 + c] : 0.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if constexpr (T::CVT) {
            float tot[MT];
#pragma unroll
            for (int c = 0; c < MT; ++c) tot[c] = 0.f;
            bool alive = true;
            for (int u = 0; u < units && alive; ++u) {
                const int a = u % NACC;
                const int g = p.grouped ? (kb0 / p.kb_per_unit + u) : 0;
                float sc = 0.f, of = 0.f;
                if (n_ok) {
                    sc = load_as_float(p.scale, p.sc_type, (size_t)g * p.N + n);
                    if (p.offset) of = load_as_float(p.offset, p.sc_type, (size_t)g * p.N + n);
                }
                if (!mbar_wait(bar_acc_full(a), (u / NACC) & 1, abort_flag, 5)) { alive = false; break; }
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < MT; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + a * MT + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float acc = __uint_as_float(v[j]);
                        if (use_xs) acc -= of * xs_sm[u * MT + c0 + j];
                        tot[c0 + j] = fmaf(sc, acc, tot[c0 + j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty(a));
            }
            if (alive && n_ok) {
                if (p.partial) {
                    float *dst = (float *)p.partial + (size_t)blockIdx.z * p.M * p.N;
#pragma unroll
                    for (int c = 0; c < MT; ++c)
                        if (m0 + c < p.M) dst[(size_t)(m0 + c) * p.N + n] = tot[c];
                } else {
                    const float b = p.bias ? load_as_float(p.bias, p.bias_type, n) : 0.f;
#pragma unroll
                    for (int c = 0; c < MT; ++c)
                        if (m0 + c < p.M) store_from_float(p.out, p.out_type, (size_t)(m0 + c) * p.N + n, tot[c] + b);
                }
            }
        } else {
            // W8A8: one accumulation over the whole K slice, exact int32.
            if (mbar_wait(bar_acc_full(0), 0, abort_flag, 5)) {
                tc_fence_after();
                float sc = 0.f;
                int bi = 0;
                if (n_ok && !p.partial && p.epilogue == EPI_DEQ_I32) {
                    sc = load_as_float(p.scale, p.sc_type, n);
                    if (p.bias) bi = ((const int32_t *)p.bias)[n];
                }
#pragma unroll 1
                for (int c0 = 0; c0 < MT; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
                    if (!n_ok) continue;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c0 + j;
                        if (m >= p.M) continue;
                        const size_t o = (size_t)m * p.N + n;
                        const int acc = (int)v[j];
                        if (p.partial) ((int32_t *)p.partial)[(size_t)blockIdx.z * p.M * p.N + o] = acc;
                        else if (p.epilogue == EPI_RAW_I32) ((int32_t *)p.out)[o] = acc;
                        else {
                            float f = (float)(acc + bi) * sc;
                            if (p.pertoken) f = f * p.pertoken[m];
                            store_from_float(p.out, p.out_type, o, f);
                        }
                    }
                }
                tc_fence_before();
            }
        }
    } else {
        // ---------------------------------------------------------------- converters (weight-only modes)
        if constexpr (T::CVT) {
            const int t = threadIdx.x - 192;          // 0..127
            const int row8 = t & 7;                   // row inside a group of 8 K-rows
            constexpr int PARTS = T::Q4 ? 4 : 8;      // 16-byte chunks per staged row
            constexpr int TASKS = T::Q4 ? 2 : 4;      // chunks per thread per K block
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(bar_full(s), (i / STAGES) & 1, abort_flag, 6)) break;
                const uint32_t src = w_stage(s), dst = w_tile(s);
#pragma unroll
                for (int task = 0; task < TASKS; ++task) {
                    const int uidx = (t >> 3) + 16 * task;
                    const int rg = uidx / PARTS, part = uidx % PARTS;
                    const int k = rg * 8 + row8;
                    uint32_t w0, w1, w2, w3;
                    if constexpr (T::Q4) {
                        // staged rows are 64 B, TMA 64-byte swizzle: chunk ^= (row / 2) % 4
                        const uint32_t a = src + k * 64 + ((part ^ ((k >> 1) & 3)) << 4);
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(a));
                    } else {
                        const uint32_t a = src + k * 128 + ((part ^ (k & 7)) << 4);
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(a));
                    }
                    const uint32_t words[4] = {w0, w1, w2, w3};
                    if constexpr (T::Q4) {
                        // one word = 8 columns -> one 16-byte chunk of 8 integers (lane order 0,4,1,5,2,6,3,7)
                        constexpr uint32_t MAGIC = T::BF16 ? 0x43004300u : 0x64006400u;  // 128.0 | 1024.0
                        constexpr uint32_t BIAS = T::BF16 ? 0x43084308u : 0x64086408u;   // 136.0 | 1032.0
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t uq = words[j] ^ 0x88888888u;  // two's complement nibble -> value + 8
                            uint32_t o[4];
#pragma unroll
                            for (int h = 0; h < 4; ++h) {
                                const uint32_t pair = ((uq >> (4 * h)) & 0x000F000Fu) | MAGIC;
                                if constexpr (T::BF16) {
                                    __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&pair),
                                                               *reinterpret_cast<const __nv_bfloat162 *>(&BIAS));
                                    o[h] = *reinterpret_cast<uint32_t *>(&d);
                                } else {
                                    __half2 d = __hsub2(*reinterpret_cast<const __half2 *>(&pair), *reinterpret_cast<const __half2 *>(&BIAS));
                                    o[h] = *reinterpret_cast<uint32_t *>(&d);
                                }
                            }
                            const int n8 = part * 4 + j;  // 16-byte chunk index along n (0..15)
                            const uint32_t a = dst + (n8 >> 3) * T::W_LBO + k * 128 + (((n8 & 7) ^ (k & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                        }
                    } else {
                        // 16 bytes = 16 columns -> two chunks of 8 integers, natural order
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            uint32_t o[4];
#pragma unroll
                            for (int h = 0; h < 4; ++h) {
                                const uint32_t ub = words[2 * j + (h >> 1)] ^ 0x80808080u;  // value + 128 per byte
                                const int b0 = (h & 1) * 2;
                                const float f0 = __uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7540 | b0)) - 8388736.f;
                                const float f1 = __uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7540 | (b0 + 1))) - 8388736.f;
                                if constexpr (T::BF16) {
                                    __nv_bfloat162 d = __floats2bfloat162_rn(f0, f1);
                                    o[h] = *reinterpret_cast<uint32_t *>(&d);
                                } else {
                                    __half2 d = __floats2half2_rn(f0, f1);
                                    o[h] = *reinterpret_cast<uint32_t *>(&d);
                                }
                            }
                            const int n8 = part * 2 + j;
                            const uint32_t a = dst + (n8 >> 3) * T::W_LBO + k * 128 + (((n8 & 7) ^ (k & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                        }
                    }
                }
                fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_wready(s));
            }
        }
    }

    // ---------------------------------------------------------------- common exit
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Activation sums per fold unit: out[u][m] = sum_{k in unit u} x[m][k]   (fp32).
__global__ void xsum_kernel(const void *x, int x_type, int M, int K, int rows_per_unit, float *out) {
    const int u = blockIdx.x, m = blockIdx.y;
    const int k0 = u * rows_per_unit, k1 = min(K, k0 + rows_per_unit);
    float s = 0.f;
    for (int k = k0 + threadIdx.x; k < k1; k += blockDim.x) s += load_as_float(x, x_type, (size_t)m * K + k);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    __shared__ float red[4];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) out[(size_t)u * M + m] = red[0] + red[1] + red[2] + red[3];
}

// Split-K reduction + epilogue: out = epi(sum_z partial[z]).
__global__ void tc_finalize_kernel(TcParams p, int split) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, mn = (size_t)p.M * p.N;
    if (i >= mn) return;
    const int n = (int)(i % p.N), m = (int)(i / p.N);
    if (p.epilogue == EPI_PLAIN) {
        float v = 0.f;
        for (int z = 0; z < split; ++z) v += ((const float *)p.partial)[z * mn + i];
        if (p.bias) v += load_as_float(p.bias, p.bias_type, n);
        store_from_float(p.out, p.out_type, i, v);
        return;
    }
    int acc = 0;
    for (int z = 0; z < split; ++z) acc += ((const int32_t *)p.partial)[z * mn + i];
    if (p.epilogue == EPI_RAW_I32) { ((int32_t *)p.out)[i] = acc; return; }
    if (p.bias) acc += ((const int32_t *)p.bias)[n];
    float f = (float)acc * load_as_float(p.scale, p.sc_type, n);
    if (p.pertoken) f = f * p.pertoken[m];
    store_from_float(p.out, p.out_type, i, f);
}

// ------------------------------------------------------------------------------------------------ host
bool device_is_sm100() {
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] { for (int &c : cached) c = -1; });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    dev &= 63;
    if (cached[dev] < 0) {
        int major = 0, minor = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return false;
        cached[dev] = (major == 10 && minor == 0) ? 1 : 0;
    }
    return cached[dev] == 1;
}

int wmode_of(const MatmulArgs &p) {
    if (p.b_type == ET_I8 && p.a_type == ET_I8) return W_I8;
    const bool bf = p.a_type == ET_BF16;
    if (p.b_type == ET_I4) return bf ? W_Q4_BF16 : W_Q4_F16;
    return bf ? W_Q8_BF16 : W_Q8_F16;
}

struct TcPlan {
    int wmode, mt, bk, split, num_kb, kb_per_split, kb_per_unit, units_total, grouped;
    bool need_xsum;
    uint64_t xsum_bytes, partial_bytes;
};

TcPlan make_plan(const MatmulArgs &p) {
    TcPlan pl{};
    pl.wmode = wmode_of(p);
    const bool i8 = pl.wmode == W_I8;
    pl.bk = i8 ? 128 : 64;
    const int mt_cap = i8 ? 256 : 128;
    pl.mt = 16;
    while (pl.mt < p.M && pl.mt < mt_cap) pl.mt *= 2;
    pl.num_kb = (int)((p.K + pl.bk - 1) / pl.bk);
    pl.grouped = (!i8 && p.group < p.K) ? 1 : 0;
    const int kb_per_group = pl.grouped ? (int)(p.group / pl.bk) : 1;
    const int n_tiles = (int)((p.N + TILE_N - 1) / TILE_N), m_tiles = (int)((p.M + pl.mt - 1) / pl.mt);
    const int tiles = n_tiles * m_tiles;
    // Split K until the grid covers the SMs about twice (small tiles leave room for two CTAs per SM),
    // but keep at least 4 K blocks per CTA so the pipeline has something to overlap.
    int split = 1;
    const int target = pl.mt <= 64 ? 296 : 148;
    if (tiles < target) split = (target + tiles - 1) / tiles;
    const int quantum = kb_per_group;                           // a CTA's slice is whole scale groups
    const int quanta = (pl.num_kb + quantum - 1) / quantum;
    const int min_q = (4 + quantum - 1) / quantum;              // >= 4 K blocks
    if (split > quanta / min_q) split = quanta / min_q;
    if (split < 1) split = 1;
    int q_per_split = (quanta + split - 1) / split;
    if (pl.grouped && q_per_split > MAX_UNITS) q_per_split = MAX_UNITS;  // bounded by the shared xsum table
    if (pl.grouped && (int64_t)q_per_split * pl.mt > 4096) q_per_split = 4096 / pl.mt;
    split = (quanta + q_per_split - 1) / q_per_split;
    pl.split = split;
    pl.kb_per_split = q_per_split * quantum;
    pl.kb_per_unit = pl.grouped ? kb_per_group : pl.kb_per_split;
    pl.units_total = (pl.num_kb + pl.kb_per_unit - 1) / pl.kb_per_unit;
    pl.need_xsum = !i8 && p.offset != nullptr;
    pl.xsum_bytes = pl.need_xsum ? align_up_u64((uint64_t)pl.units_total * p.M * sizeof(float), 256) : 0;
    pl.partial_bytes = split > 1 ? (uint64_t)split * p.M * p.N * 4 : 0;
    return pl;
}

template <int WMODE, int MT, int STAGES>
cudaError_t launch_one(const CUtensorMap &tx, const CUtensorMap &tw, const TcParams &tp, dim3 grid, cudaStream_t s) {
    using L = SmemLayout<WMODE, MT, STAGES>;
    auto kern = tc_kernel<WMODE, MT, STAGES>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    kern<<<grid, WTraits<WMODE>::CVT ? 320 : 192, L::TOTAL, s>>>(tx, tw, tp);
    count_launch();
    return cudaGetLastError();
}

template <int WMODE>
cudaError_t dispatch_mt(int mt, const CUtensorMap &tx, const CUtensorMap &tw, const TcParams &tp, dim3 grid, cudaStream_t s) {
    switch (mt) {
        case 16: return launch_one<WMODE, 16, 4>(tx, tw, tp, grid, s);
        case 32: return launch_one<WMODE, 32, 4>(tx, tw, tp, grid, s);
        case 64: return launch_one<WMODE, 64, 4>(tx, tw, tp, grid, s);
        case 128: return launch_one<WMODE, 128, 4>(tx, tw, tp, grid, s);
        case 256:
            if constexpr (WMODE == W_I8) return launch_one<WMODE, 256, 4>(tx, tw, tp, grid, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

// Weight-only matmuls go to the persistent stream-K kernel (wq_tc.cu) unless B200_QMM_WQ=legacy.
static bool use_stream_wq(const MatmulArgs &p) {
    if (p.epilogue != EPI_PLAIN || !p.scale) return false;
    const char *e = getenv("B200_QMM_WQ");
    if (e && !strcmp(e, "legacy")) return false;
    return wq_tc_supported(p);
}

bool tc_supported(const MatmulArgs &p) {
    if (!device_is_sm100() || !encode_fn()) return false;
    if (use_stream_wq(p)) return true;
    if (p.batch != 1 || p.b_transposed || p.accumulate || p.M < 1) return false;
    if (p.M > (1 << 24) || p.N > (1 << 24) || p.K > (1 << 24)) return false;
    auto aligned16 = [](const void *q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!aligned16(p.a) || !aligned16(p.b)) return false;
    if (p.epilogue == EPI_DEQ_I32 || p.epilogue == EPI_RAW_I32) {
        if (p.a_type != ET_I8 || p.b_type != ET_I8) return false;
        return p.K % 16 == 0 && p.N % 16 == 0;
    }
    if (p.epilogue == EPI_PLAIN && p.scale && !p.a_scale && !p.b_scale) {
        if (p.a_type != ET_F16 && p.a_type != ET_BF16) return false;
        if (p.b_type != ET_I4 && p.b_type != ET_I8) return false;
        if (p.sc_type != p.a_type || (p.bias && p.bias_type != p.a_type)) return false;
        if (p.K % 8 != 0) return false;
        if (p.b_type == ET_I4 ? (p.N % 32 != 0) : (p.N % 16 != 0)) return false;
        if (p.group < p.K && (p.group % 64 != 0 || p.K % p.group != 0)) return false;
        return true;
    }
    return false;
}

void tc_plan(MatmulArgs &p) { p.split_k = use_stream_wq(p) ? 1 : make_plan(p).split; }

uint64_t tc_workspace_bytes(const MatmulArgs &p) {
    if (use_stream_wq(p)) return wq_tc_workspace_bytes(p);
    TcPlan pl = make_plan(p);
    return pl.xsum_bytes + pl.partial_bytes;
}

cudaError_t launch_tc(const MatmulArgs &p, cudaStream_t s) {
    if (use_stream_wq(p)) return launch_wq_tc(p, s);
    const TcPlan pl = make_plan(p);
    if (p.workspace_bytes < pl.xsum_bytes + pl.partial_bytes) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15)) return cudaErrorMisalignedAddress;
    const bool i8 = pl.wmode == W_I8;

    CUtensorMap tx, tw;
    bool ok;
    if (i8) {
        ok = make_map(&tx, p.a, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.K, p.M, p.K, 128, pl.mt, CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_map(&tw, p.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.N, p.K, p.N, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        const CUtensorMapDataType xt = p.a_type == ET_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        ok = make_map(&tx, p.a, xt, p.K, p.M, p.K * 2, 64, pl.mt, CU_TENSOR_MAP_SWIZZLE_128B);
        if (p.b_type == ET_I4)
            ok = ok && make_map(&tw, p.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.N / 2, p.K, p.N / 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_64B);
        else
            ok = ok && make_map(&tw, p.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.N, p.K, p.N, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (!ok) return cudaErrorInvalidValue;

    TcParams tp{};
    tp.out = p.out;
    char *ws = (char *)p.workspace;
    tp.xsum = pl.need_xsum ? (const float *)ws : nullptr;
    tp.partial = pl.split > 1 ? (void *)(ws + pl.xsum_bytes) : nullptr;
    tp.scale = p.scale; tp.offset = p.offset; tp.bias = p.bias; tp.pertoken = p.pertoken;
    tp.sc_type = p.sc_type; tp.bias_type = p.bias_type; tp.out_type = p.out_type; tp.epilogue = p.epilogue;
    tp.M = (int)p.M; tp.N = (int)p.N; tp.K = (int)p.K;
    tp.num_kb = pl.num_kb; tp.kb_per_split = pl.kb_per_split; tp.kb_per_unit = pl.kb_per_unit; tp.grouped = pl.grouped;

    if (pl.need_xsum) {
        dim3 g(pl.units_total, (unsigned)p.M);
        xsum_kernel<<<g, 128, 0, s>>>(p.a, p.a_type, tp.M, tp.K, pl.kb_per_unit * pl.bk, (float *)ws);
        count_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    dim3 grid((unsigned)((p.N + TILE_N - 1) / TILE_N), (unsigned)((p.M + pl.mt - 1) / pl.mt), (unsigned)pl.split);
    cudaError_t e;
    switch (pl.wmode) {
        case W_I8: e = dispatch_mt<W_I8>(pl.mt, tx, tw, tp, grid, s); break;
        case W_Q4_BF16: e = dispatch_mt<W_Q4_BF16>(pl.mt, tx, tw, tp, grid, s); break;
        case W_Q4_F16: e = dispatch_mt<W_Q4_F16>(pl.mt, tx, tw, tp, grid, s); break;
        case W_Q8_BF16: e = dispatch_mt<W_Q8_BF16>(pl.mt, tx, tw, tp, grid, s); break;
        default: e = dispatch_mt<W_Q8_F16>(pl.mt, tx, tw, tp, grid, s); break;
    }
    if (e != cudaSuccess) return e;
    if (pl.split > 1) {
        const size_t mn = (size_t)p.M * p.N;
        tc_finalize_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(tp, pl.split);
        count_launch();
        e = cudaGetLastError();
    }
    return e;
}

unsigned int tc_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    const unsigned int w = wq_tc_device_status();
    return v ? v : w;
}

}  // namespace qmm
