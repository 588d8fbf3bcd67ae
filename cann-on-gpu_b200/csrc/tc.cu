// Dense tcgen05 kernel of the quantized-matmul family (sm_100a only): both operands go from HBM to
// swizzled shared memory by TMA and straight into tcgen05.mma; accumulators live in TMEM.
//
//   * The WEIGHT tile sits on the MMA's M side (128 output columns n per tile) and the ACTIVATION tile
//     on its N side (MT = 16..256 rows m).  The caller's weight is [K,N] with N contiguous, which is the
//     "MN-major" operand form of tcgen05.mma for 8- and 16-bit types, so no transpose pass exists
//     anywhere (the reference transposes the whole weight on every call, cuda/src/ops/matmul.cu:824).
//     Small M costs nothing: the instruction's N extent shrinks to 16.
//   * Accumulator layout: TMEM lane = output column n, TMEM column = output row m, so everything
//     indexed by n (scale, bias) is a per-thread scalar in the epilogue.
//   * Modes: W8A8 (kind::i8, exact int32 accumulators, fused epilogue
//     float(acc + bias) * scale[n] * pertoken[m] and cast; the reference runs an int8 GEMM into a
//     workspace and a separate scale kernel, matmul.cu:825-846) and 16-bit dense (kind::f16, bf16 or
//     fp16 operands, fp32 accumulators) used by the MX matmuls and the large-M weight-only path after
//     their operands have been expanded (dequant.cu).
//   * Persistent: gridDim.x CTAs walk the list of (tile, K slice) units; the two TMEM accumulators
//     alternate between units, so the epilogue of one unit overlaps the MMAs of the next.
//     Warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM owner), warps 2-9 = epilogue (two sets of four
//     warps, each set takes half of the accumulator columns).
//   * Whole rounds of one tile per SM run unsplit; only the tiles left over after them (all tiles
//     when there are fewer tiles than SMs) may be cut into K slices, so that the last round is
//     short instead of mostly idle.  Their raw accumulators go to the caller's workspace, one
//     [MT][128] tile per slice, and tc_finalize_kernel sums them and applies the epilogue.  Whether
//     to cut, and how finely, is decided by a small cost model (make_plan).
//   * Every wait is bounded (about a second) and records a code in a device status word.
#include <cstring>
#include <mutex>

#include "tc_common.cuh"

namespace qmm {
namespace {

enum DMode : int { D_I8 = 0, D_BF16, D_F16 };

template <int MODE> struct DTraits;
// K rows per stage, K per MMA, bytes between MMA K steps inside the weight tile, pitch of the two
// 64-column halves of a 16-bit weight tile.
template <> struct DTraits<D_I8>   { static constexpr int BK = 128, UMMA_K = 32, W_KSTEP = 4096, W_LBO = 16384; };
template <> struct DTraits<D_BF16> { static constexpr int BK = 64,  UMMA_K = 16, W_KSTEP = 2048, W_LBO = 8192; };
template <> struct DTraits<D_F16>  { static constexpr int BK = 64,  UMMA_K = 16, W_KSTEP = 2048, W_LBO = 8192; };

constexpr int TILE_N = 128;          // output columns per tile = MMA M
constexpr int W_TILE_BYTES = 16384;  // weight tile per stage: 128 n x 128 k int8, or 2 x (64 n x 64 k) 16-bit

struct TcParams {
    void *out;
    void *partial;            // [split][tail tile][MT][128] fp32 or int32 raw accumulators of the split tiles, or null
    const void *scale;        // W8A8: [N]
    const void *bias;
    const float *pertoken;
    int sc_type, bias_type, out_type, epilogue;
    int M, N, K;
    int m_tiles, tiles;       // tiles are numbered n_tile * m_tiles + m_tile
    int num_kb;               // K blocks in total
    int full_units;           // the first full_units tiles run unsplit, one unit each (a multiple of the grid)
    int tail_tiles;           // the remaining tiles ...
    int split;                // ... are cut into `split` K slices each, so the last round is short
    int kb_per_split;         // K blocks per slice of a tail tile
    int units;                // full_units + tail_tiles * split
    int mt, tn;               // rows and columns per tile (for the finalize kernel)
};

template <int MT, int STAGES>
struct DSmem {
    static constexpr int X_BYTES = MT * 128;
    static constexpr int STAGE_BYTES = X_BYTES + W_TILE_BYTES;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 4;
    static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
    static constexpr int TOTAL = MISC_OFF + 16 + 1024;  // + slack for the 1024-byte base alignment
};

template <int MODE, int MT, int STAGES>
__global__ void __launch_bounds__(320, 1)
tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const TcParams p) {
    using T = DTraits<MODE>;
    using L = DSmem<MT, STAGES>;
    constexpr bool INT8 = (MODE == D_I8);
    constexpr int TMEM_COLS = (2 * MT) < 32 ? 32 : (2 * MT);  // two accumulators; powers of two by construction
    constexpr int KSTEPS = T::BK / T::UMMA_K;
    constexpr uint32_t IDESC = INT8 ? instr_desc(2, 1, TILE_N, MT) : instr_desc(1, MODE == D_BF16 ? 1 : 0, TILE_N, MT);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    auto x_tile = [&](int s) { return base + s * L::STAGE_BYTES; };
    auto w_tile = [&](int s) { return base + s * L::STAGE_BYTES + L::X_BYTES; };
    auto bar_full = [&](int s) { return base + L::BAR_OFF + 8 * s; };
    auto bar_empty = [&](int s) { return base + L::BAR_OFF + 8 * (STAGES + s); };
    auto bar_acc_full = [&](int a) { return base + L::BAR_OFF + 8 * (2 * STAGES + a); };
    auto bar_acc_empty = [&](int a) { return base + L::BAR_OFF + 8 * (2 * STAGES + 2 + a); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen_base + L::MISC_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + L::MISC_OFF + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(bar_acc_full(a), 1); mbar_init(bar_acc_empty(a), 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void *)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched with programmatic stream serialisation: everything above (barriers, tensor-memory allocation) may run
    // while the kernel before this one in the stream is still finishing; nothing below touches global memory before
    // that kernel has completed and its writes are visible.  Without the launch attribute both instructions do nothing.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // unit u -> (K slice z, tile); tiles of one K slice are consecutive and m-tiles of one weight tile
    // are adjacent, so CTAs running side by side share weight tiles in L2.
    // z < 0: the unit is a whole tile and runs the epilogue itself; z >= 0: K slice z of tail tile
    // (tile - full_units), whose raw accumulators go to the workspace.
    auto unit_geom = [&](int u, int &n0, int &m0, int &kb0, int &nkb, int &z) {
        int tile;
        if (u < p.full_units) {
            tile = u; z = -1; kb0 = 0; nkb = p.num_kb;
        } else {
            const int v = u - p.full_units;
            tile = p.full_units + v % p.tail_tiles;
            z = v / p.tail_tiles;
            kb0 = z * p.kb_per_split;
            nkb = min(p.num_kb, kb0 + p.kb_per_split) - kb0;
            if (p.split == 1) z = -1;
        }
        n0 = (tile / p.m_tiles) * TILE_N;
        m0 = (tile % p.m_tiles) * MT;
    };

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
                int n0, m0, kb0, nkb, z;
                unit_geom(u, n0, m0, kb0, nkb, z);
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(bar_empty(s), ((it / STAGES) - 1) & 1, abort_flag, 1)) { ok = false; break; }
                    mbar_expect_tx(bar_full(s), L::STAGE_BYTES);
                    const int k = (kb0 + i) * T::BK;
                    tma_load_2d(x_tile(s), &tm_x, bar_full(s), k, m0);
                    if constexpr (INT8) {
                        tma_load_2d(w_tile(s), &tm_w, bar_full(s), n0, k);
                    } else {
                        tma_load_2d(w_tile(s), &tm_w, bar_full(s), n0, k);                   // columns n0 .. n0+63
                        tma_load_2d(w_tile(s) + T::W_LBO, &tm_w, bar_full(s), n0 + 64, k);   // columns n0+64 .. n0+127
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int it = 0, ui = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++ui) {
                int n0, m0, kb0, nkb, z;
                unit_geom(u, n0, m0, kb0, nkb, z);
                const int a = ui & 1;
                if (ui >= 2) {
                    if (!mbar_wait(bar_acc_empty(a), ((ui >> 1) - 1) & 1, abort_flag, 2)) { ok = false; break; }
                    tc_fence_after();  // the epilogue's TMEM reads of this accumulator are complete
                }
                const uint32_t d = tmem_base + a * MT;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(bar_full(s), (it / STAGES) & 1, abort_flag, 3)) { ok = false; break; }
#pragma unroll
                    for (int kk = 0; kk < KSTEPS; ++kk) {
                        const uint64_t a_desc = smem_desc(w_tile(s) + kk * T::W_KSTEP, T::W_LBO, 1024);
                        const uint64_t b_desc = smem_desc(x_tile(s) + kk * 32, 16, 1024);
                        tc_mma<INT8>(d, a_desc, b_desc, IDESC, (i > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty(s));
                }
                if (ok) tc_commit(bar_acc_full(a));
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (two sets x four warps)
        const int eset = (warp - 2) >> 2;             // which half of the accumulator columns
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int r = q * 32 + lane;                  // accumulator lane = output column inside the tile
        constexpr int CH = MT >= 32 ? MT / 2 : MT;    // columns per set (a 16-row tile is not split)
        const bool active = MT >= 32 || eset == 0;
        const int cb = MT >= 32 ? eset * CH : 0;
        int ui = 0;
        for (int u = blockIdx.x; u < p.units; u += gridDim.x, ++ui) {
            int n0, m0, kb0, nkb, z;
            unit_geom(u, n0, m0, kb0, nkb, z);
            const int a = ui & 1;
            const int n = n0 + r;
            const bool n_ok = n < p.N;
            const bool to_partial = z >= 0;
            uint32_t *part_tile = nullptr;   // this unit's [MT][128] raw tile in the workspace
            if (to_partial) {
                const int tail_idx = (u - p.full_units) % p.tail_tiles;
                part_tile = (uint32_t *)p.partial + ((size_t)z * p.tail_tiles + tail_idx) * (MT * TILE_N);
            }
            float sc = 0.f, bf = 0.f;
            int bi = 0;
            if (n_ok && !to_partial) {
                if (p.epilogue == EPI_DEQ_I32) {
                    sc = load_as_float(p.scale, p.sc_type, n);
                    if (p.bias) bi = ((const int32_t *)p.bias)[n];
                } else if (p.epilogue == EPI_PLAIN && p.bias) {
                    bf = load_as_float(p.bias, p.bias_type, n);
                }
            }
            // per-token scales of this set's rows: lane l keeps rows cb + l, cb + l + 32, ... and hands them
            // out with shuffles, so the column loop issues no dependent global loads
            constexpr int PR = (CH + 31) / 32;
            float ptv[PR];
#pragma unroll
            for (int i = 0; i < PR; ++i) {
                const int m = m0 + cb + lane + 32 * i;
                ptv[i] = (p.pertoken && lane + 32 * i < CH && m < p.M) ? __ldg(p.pertoken + m) : 1.f;
            }
            const bool has_pt = p.pertoken != nullptr;
            if (!mbar_wait(bar_acc_full(a), (ui >> 1) & 1, abort_flag, 5)) break;
            tc_fence_after();
            if (active && to_partial) {
                // K slice of a tail tile: raw fp32 / int32 bits of the whole tile go to the workspace
#pragma unroll 1
                for (int c0 = cb; c0 < cb + CH; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + a * MT + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) part_tile[(c0 + j) * TILE_N + r] = v[j];
                }
            } else if (active) {
#pragma unroll 1
                for (int c0 = cb; c0 < cb + CH; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + a * MT + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int cl = c0 - cb + j;
                        const float pt = has_pt ? __shfl_sync(0xffffffffu, ptv[cl >> 5], cl & 31) : 1.f;
                        const int m = m0 + c0 + j;
                        if (!n_ok || m >= p.M) continue;
                        const size_t o = (size_t)m * p.N + n;
                        if constexpr (INT8) {
                            const int acc = (int)v[j];
                            if (p.epilogue == EPI_RAW_I32) ((int32_t *)p.out)[o] = acc;
                            else {
                                float f = (float)(acc + bi) * sc;
                                if (has_pt) f = f * pt;
                                store_from_float(p.out, p.out_type, o, f);
                            }
                        } else {
                            // optional per-row scale (1 without): fmaf(acc, 1, bias) rounds like acc + bias
                            store_from_float(p.out, p.out_type, o, fmaf(__uint_as_float(v[j]), pt, bf));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(a));
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

// ------------------------------------------------------------------------------------------------
// Row-tile variant for many rows (M > 128): the ACTIVATION tile (128 rows m) sits on the MMA's M side
// and the WEIGHT tile (256 columns n, still MN-major straight from the caller's [K,N]) on its N side,
// so TMEM lane = output row and a thread holds consecutive output columns: the epilogue packs them
// and writes 16 bytes per store instead of one 2-byte store per element.  With short K (W8A8,
// K = 4096) the column-per-lane epilogue above takes longer than the unit's MMAs and sets the pace
// (measured: 17-21 us per 256 x 128 tile against 14 us of MMAs); this one does not.
// Same warp roles, unit list, K-split tail and bounded waits as tc_kernel.
constexpr int RT_M = 128, RT_N = 256;

template <int STAGES>
struct RSmem {
    static constexpr int X_BYTES = RT_M * 128;
    static constexpr int W_BYTES = RT_N * 128;
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 4;
    static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
    static constexpr int COL_OFF = MISC_OFF + 16;           // scale[256] then bias[256] of the current tile
    static constexpr int TOTAL = COL_OFF + 2 * RT_N * 4 + 1024;
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

enum ROut : int { RO_BF16 = 0, RO_F16, RO_F32, RO_RAW };

// One row's 128 accumulator columns [cb, cb + 128) of a tile -> out[m][n0 + cb ...], 8 columns per
// step.  sc_s / bi_s hold the tile's per-column scale and bias (float bits in bi_s for the 16-bit modes).
template <bool INT8, int OUT>
__device__ __forceinline__ void rt_store_row(uint32_t taddr, const TcParams &p, const float *sc_s, const int32_t *bi_s, int cb, int n0,
                                             int m, bool m_ok, float pt) {
    constexpr int ESZ = (OUT == RO_BF16 || OUT == RO_F16) ? 2 : 4;
    uint8_t *orow = (uint8_t *)p.out + ((size_t)m * p.N + n0 + cb) * ESZ;
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(taddr + c0, v);
        if (!m_ok) continue;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int c = c0 + 8 * g;
            if (n0 + cb + c >= p.N) break;   // N is a multiple of 8 on this path
            const float4 s0 = *reinterpret_cast<const float4 *>(sc_s + cb + c), s1 = *reinterpret_cast<const float4 *>(sc_s + cb + c + 4);
            const int4 b0 = *reinterpret_cast<const int4 *>(bi_s + cb + c), b1 = *reinterpret_cast<const int4 *>(bi_s + cb + c + 4);
            const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const int bi[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            if constexpr (OUT == RO_RAW) {
                uint4 *o = reinterpret_cast<uint4 *>(orow + (size_t)c * 4);
                o[0] = make_uint4(v[8 * g], v[8 * g + 1], v[8 * g + 2], v[8 * g + 3]);
                o[1] = make_uint4(v[8 * g + 4], v[8 * g + 5], v[8 * g + 6], v[8 * g + 7]);
            } else {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if constexpr (INT8) f[j] = ((float)((int)v[8 * g + j] + bi[j]) * sc[j]) * pt;   // pt is 1 without per-token scales
                    else f[j] = fmaf(__uint_as_float(v[8 * g + j]), pt, __int_as_float(bi[j]));   // pt: optional per-row scale
                }
                if constexpr (OUT == RO_F32) {
                    float4 *o = reinterpret_cast<float4 *>(orow + (size_t)c * 4);
                    o[0] = make_float4(f[0], f[1], f[2], f[3]);
                    o[1] = make_float4(f[4], f[5], f[6], f[7]);
                } else {
                    uint4 o;
                    if constexpr (OUT == RO_BF16) {
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(f[0], f[1]), h1 = __floats2bfloat162_rn(f[2], f[3]),
                                       h2 = __floats2bfloat162_rn(f[4], f[5]), h3 = __floats2bfloat162_rn(f[6], f[7]);
                        o = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                       *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                    } else {
                        __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]), h2 = __floats2half2_rn(f[4], f[5]),
                                h3 = __floats2half2_rn(f[6], f[7]);
                        o = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                       *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                    }
                    *reinterpret_cast<uint4 *>(orow + (size_t)c * 2) = o;
                }
            }
        }
    }
}

template <int MODE, int STAGES>
__global__ void __launch_bounds__(320, 1)
tc_rowtile_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const TcParams p) {
    using T = DTraits<MODE>;
    using L = RSmem<STAGES>;
    constexpr bool INT8 = (MODE == D_I8);
    constexpr int TMEM_COLS = 2 * RT_N;
    constexpr int KSTEPS = T::BK / T::UMMA_K;
    constexpr int W_BOXES = INT8 ? 2 : 4;              // 128-byte-wide column blocks of the weight tile
    constexpr int W_BOX_COLS = INT8 ? 128 : 64;
    // A = activations, K-major; B = weights, MN-major; M = 128, N = 256
    constexpr uint32_t IDESC = (INT8 ? instr_desc(2, 1, RT_M, RT_N) : instr_desc(1, MODE == D_BF16 ? 1 : 0, RT_M, RT_N)) ^ (1u << 15) ^ (1u << 16);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    auto x_tile = [&](int s) { return base + s * L::STAGE_BYTES; };
    auto w_tile = [&](int s) { return base + s * L::STAGE_BYTES + L::X_BYTES; };
    auto bar_full = [&](int s) { return base + L::BAR_OFF + 8 * s; };
    auto bar_empty = [&](int s) { return base + L::BAR_OFF + 8 * (STAGES + s); };
    auto bar_acc_full = [&](int a) { return base + L::BAR_OFF + 8 * (2 * STAGES + a); };
    auto bar_acc_empty = [&](int a) { return base + L::BAR_OFF + 8 * (2 * STAGES + 2 + a); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen_base + L::MISC_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + L::MISC_OFF + 4);
    float *sc_s = reinterpret_cast<float *>(gen_base + L::COL_OFF);
    int32_t *bi_s = reinterpret_cast<int32_t *>(sc_s + RT_N);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(bar_acc_full(a), 1); mbar_init(bar_acc_empty(a), 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void *)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Same unit list as tc_kernel; a tile is 128 rows x 256 columns here.
    auto unit_geom = [&](int u, int &n0, int &m0, int &kb0, int &nkb, int &z) {
        int tile;
        if (u < p.full_units) {
            tile = u; z = -1; kb0 = 0; nkb = p.num_kb;
        } else {
            const int v = u - p.full_units;
            tile = p.full_units + v % p.tail_tiles;
            z = v / p.tail_tiles;
            kb0 = z * p.kb_per_split;
            nkb = min(p.num_kb, kb0 + p.kb_per_split) - kb0;
            if (p.split == 1) z = -1;
        }
        n0 = (tile / p.m_tiles) * RT_N;
        m0 = (tile % p.m_tiles) * RT_M;
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
                int n0, m0, kb0, nkb, z;
                unit_geom(u, n0, m0, kb0, nkb, z);
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(bar_empty(s), ((it / STAGES) - 1) & 1, abort_flag, 1)) { ok = false; break; }
                    mbar_expect_tx(bar_full(s), L::STAGE_BYTES);
                    const int k = (kb0 + i) * T::BK;
                    tma_load_2d(x_tile(s), &tm_x, bar_full(s), k, m0);
#pragma unroll
                    for (int j = 0; j < W_BOXES; ++j) tma_load_2d(w_tile(s) + j * T::W_LBO, &tm_w, bar_full(s), n0 + j * W_BOX_COLS, k);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, ui = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++ui) {
                int n0, m0, kb0, nkb, z;
                unit_geom(u, n0, m0, kb0, nkb, z);
                const int a = ui & 1;
                if (ui >= 2) {
                    if (!mbar_wait(bar_acc_empty(a), ((ui >> 1) - 1) & 1, abort_flag, 2)) { ok = false; break; }
                    tc_fence_after();
                }
                const uint32_t d = tmem_base + a * RT_N;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(bar_full(s), (it / STAGES) & 1, abort_flag, 3)) { ok = false; break; }
#pragma unroll
                    for (int kk = 0; kk < KSTEPS; ++kk) {
                        const uint64_t a_desc = smem_desc(x_tile(s) + kk * 32, 16, 1024);
                        const uint64_t b_desc = smem_desc(w_tile(s) + kk * T::W_KSTEP, T::W_LBO, 1024);
                        tc_mma<INT8>(d, a_desc, b_desc, IDESC, (i > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty(s));
                }
                if (ok) tc_commit(bar_acc_full(a));
            }
        }
    } else {
        // epilogue: warp's TMEM lane quarter = 32 rows; the two sets of four warps take 128 columns each
        const int te = threadIdx.x - 64;
        const int eset = (warp - 2) >> 2, q = warp & 3;
        const int row = q * 32 + lane, cb = eset * 128;
        int ui = 0;
        for (int u = blockIdx.x; u < p.units; u += gridDim.x, ++ui) {
            int n0, m0, kb0, nkb, z;
            unit_geom(u, n0, m0, kb0, nkb, z);
            const int a = ui & 1;
            const bool to_partial = z >= 0;
            const int m = m0 + row;
            const bool m_ok = m < p.M;
            epi_bar_sync();   // every warp is done with the previous tile's scale and bias
            {
                const int n = n0 + te;
                float sc = 0.f;
                int bi = 0;
                if (n < p.N && !to_partial) {
                    if (p.epilogue == EPI_DEQ_I32) {
                        sc = load_as_float(p.scale, p.sc_type, n);
                        if (p.bias) bi = ((const int32_t *)p.bias)[n];
                    } else if (p.epilogue == EPI_PLAIN && p.bias) {
                        bi = __float_as_int(load_as_float(p.bias, p.bias_type, n));
                    }
                }
                sc_s[te] = sc;
                bi_s[te] = bi;
            }
            const float pt = (p.pertoken && m_ok && !to_partial) ? __ldg(p.pertoken + m) : 1.f;
            epi_bar_sync();
            if (!mbar_wait(bar_acc_full(a), (ui >> 1) & 1, abort_flag, 5)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * RT_N + cb;
            if (to_partial) {
                // K slice of a tail tile: the raw [128][256] accumulators go to the workspace
                const int tail_idx = (u - p.full_units) % p.tail_tiles;
                uint32_t *prow = (uint32_t *)p.partial + ((size_t)z * p.tail_tiles + tail_idx) * (RT_M * RT_N) + (size_t)row * RT_N + cb;
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c0, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<uint4 *>(prow + c0)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            } else if (p.epilogue == EPI_RAW_I32) {
                rt_store_row<INT8, RO_RAW>(taddr, p, sc_s, bi_s, cb, n0, m, m_ok, pt);
            } else if (p.out_type == ET_BF16) {
                rt_store_row<INT8, RO_BF16>(taddr, p, sc_s, bi_s, cb, n0, m, m_ok, pt);
            } else if (p.out_type == ET_F16) {
                rt_store_row<INT8, RO_F16>(taddr, p, sc_s, bi_s, cb, n0, m, m_ok, pt);
            } else {
                rt_store_row<INT8, RO_F32>(taddr, p, sc_s, bi_s, cb, n0, m, m_ok, pt);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(a));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Split-K reduction + epilogue: out = epi(sum_z partial[z]).
__global__ void tc_finalize_kernel(TcParams p) {
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x, per_tile = (size_t)p.mt * p.tn;
    if (e >= per_tile * p.tail_tiles) return;
    const int t = (int)(e / per_tile), ml = (int)((e / p.tn) % p.mt), nl = (int)(e % p.tn);
    const int tile = p.full_units + t;
    const int n = (tile / p.m_tiles) * p.tn + nl, m = (tile % p.m_tiles) * p.mt + ml;
    if (n >= p.N || m >= p.M) return;
    const size_t i = (size_t)m * p.N + n, stride = per_tile * p.tail_tiles, off = e;
    if (p.epilogue == EPI_PLAIN) {
        float v = 0.f;
        for (int z = 0; z < p.split; ++z) v += ((const float *)p.partial)[z * stride + off];
        if (p.pertoken) v *= p.pertoken[m];
        if (p.bias) v += load_as_float(p.bias, p.bias_type, n);
        store_from_float(p.out, p.out_type, i, v);
        return;
    }
    int acc = 0;
    for (int z = 0; z < p.split; ++z) acc += ((const int32_t *)p.partial)[z * stride + off];
    if (p.epilogue == EPI_RAW_I32) { ((int32_t *)p.out)[i] = acc; return; }
    if (p.bias) acc += ((const int32_t *)p.bias)[n];
    float f = (float)acc * load_as_float(p.scale, p.sc_type, n);
    if (p.pertoken) f = f * p.pertoken[m];
    store_from_float(p.out, p.out_type, i, f);
}

// ------------------------------------------------------------------------------------------------ host
thread_local int g_reserved_sms = 0;
struct DevInfo { int sm100 = -1, sms = 0; };

DevInfo &dev_info() {
    static DevInfo info[64];
    static DevInfo none;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return none;
    DevInfo &d = info[dev & 63];
    if (d.sm100 < 0) {
        int major = 0, minor = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return none;
        d.sms = sms;
        d.sm100 = (major == 10 && minor == 0) ? 1 : 0;
    }
    return d;
}

struct TcPlan {
    int mode, mt, tn, bk, split, num_kb, kb_per_split, m_tiles, tiles, units, P, full_units, tail_tiles;
    bool rowtile;
    uint64_t partial_bytes;
};

TcPlan make_plan(const MatmulArgs &p) {
    TcPlan pl{};
    pl.mode = p.a_type == ET_I8 ? D_I8 : (p.a_type == ET_BF16 ? D_BF16 : D_F16);
    pl.bk = pl.mode == D_I8 ? 128 : 64;
    pl.mt = 16;
    while (pl.mt < p.M && pl.mt < 256) pl.mt *= 2;
    pl.tn = TILE_N;
    // Many rows: 128-row x 256-column tiles with the rows on the accumulator lanes (tc_rowtile_kernel),
    // where the output type allows its 16-byte stores (an output pointer off that alignment is refused at
    // launch).  B200_QMM_DENSE_ROWTILE=0 keeps the column-per-lane kernel.
    pl.rowtile = false;
    if (p.M > 128 && p.N % 8 == 0) {
        const bool out_ok = p.epilogue == EPI_RAW_I32 ? p.out_type == ET_I32
                                                      : (p.out_type == ET_BF16 || p.out_type == ET_F16 || p.out_type == ET_F32);
        const char *e = getenv("B200_QMM_DENSE_ROWTILE");
        pl.rowtile = out_ok && !(e && atoi(e) == 0);
    }
    if (pl.rowtile) { pl.mt = RT_M; pl.tn = RT_N; }
    pl.num_kb = (int)((p.K + pl.bk - 1) / pl.bk);
    const int n_tiles = (int)((p.N + pl.tn - 1) / pl.tn);
    pl.m_tiles = (int)((p.M + pl.mt - 1) / pl.mt);
    pl.tiles = n_tiles * pl.m_tiles;
    int sms = dev_info().sms > 0 ? dev_info().sms : 148;
    // SMs the caller wants left free for a kernel that runs beside this one (aclnnB200ReserveSms): a persistent
    // kernel on every SM would keep a concurrent collective from starting until it has finished.
    if (g_reserved_sms > 0) sms = sms - g_reserved_sms > 8 ? sms - g_reserved_sms : 8;
    // Whole rounds of one tile per SM run unsplit.  The tiles left over (all of them when there are
    // fewer tiles than SMs) are cut along K so that the last round is short instead of leaving most
    // SMs idle -- but only where that pays.  A unit pulls kb * bk * (mt + 128) operand bytes into its SM
    // at about 45 GB/s (what one SM gets when all of them stream), units run in rounds of one per SM, and
    // a split adds the raw partial tiles (written, then read by the finalize kernel, at about 3 TB/s)
    // plus that kernel's launch.  Take the split with the smallest estimate, keeping at least 4 K
    // blocks per unit.  (Measured on W8A8 4096 x 14336: M = 1 takes 14.0 us unsplit and 18.4 us split in
    // 3; M = 256 takes 34 us unsplit and 59 us split in 3.)  B200_QMM_DENSE_SPLIT=<n> overrides.
    pl.full_units = (pl.tiles / sms) * sms;
    pl.tail_tiles = pl.tiles - pl.full_units;
    int split = 1;
    if (pl.tail_tiles > 0) {
        const double elem = pl.mode == D_I8 ? 1.0 : 2.0;
        double best = 1e30;
        const int max_split = pl.num_kb / 4 > 1 ? pl.num_kb / 4 : 1;
        for (int sct = 1; sct <= max_split && sct <= 64; ++sct) {
            const int kbps = (pl.num_kb + sct - 1) / sct, eff = (pl.num_kb + kbps - 1) / kbps;
            const long long units = (long long)pl.tail_tiles * eff;
            const double rounds = (double)((units + sms - 1) / sms);
            double t = rounds * kbps * pl.bk * (pl.mt + pl.tn) * elem / 45e9;
            if (eff > 1) t += 2.0 * eff * (double)pl.tail_tiles * pl.mt * pl.tn * 4.0 / 3e12 + 3e-6;
            if (t < best * 0.97) { best = t; split = eff; }   // a later split must win by a margin
        }
        if (const char *e = getenv("B200_QMM_DENSE_SPLIT")) { const int v = atoi(e); if (v >= 1) split = v; }
        if (split > pl.num_kb) split = pl.num_kb;
        if (split < 1) split = 1;
    }
    pl.kb_per_split = (pl.num_kb + split - 1) / split;
    pl.split = (pl.num_kb + pl.kb_per_split - 1) / pl.kb_per_split;
    pl.units = pl.full_units + pl.tail_tiles * pl.split;
    pl.P = pl.units < sms ? pl.units : sms;
    pl.partial_bytes = pl.split > 1 ? (uint64_t)pl.split * pl.tail_tiles * pl.mt * pl.tn * 4 : 0;
    return pl;
}

template <int MODE, int MT, int STAGES>
cudaError_t launch_one(const CUtensorMap &tx, const CUtensorMap &tw, const TcParams &tp, int P, cudaStream_t s) {
    using L = DSmem<MT, STAGES>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA");
    auto kern = tc_kernel<MODE, MT, STAGES>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    // Programmatic stream serialisation (see the kernel's start-up): at decode shapes the call is a few microseconds
    // long and its start-up is a visible part of that.  B200_QMM_PDL=0 launches the plain way.
    static const int pdl = [] { const char *e = getenv("B200_QMM_PDL"); return e ? atoi(e) : 1; }();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)P);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = (size_t)L::TOTAL;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl >= 1 ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tx, tw, tp);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <int MODE>
cudaError_t launch_rowtile(const CUtensorMap &tx, const CUtensorMap &tw, const TcParams &tp, int P, cudaStream_t s) {
    using L = RSmem<4>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA");
    auto kern = tc_rowtile_kernel<MODE, 4>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    kern<<<P, 320, L::TOTAL, s>>>(tx, tw, tp);
    count_launch();
    return cudaGetLastError();
}

template <int MODE>
cudaError_t dispatch_mt(int mt, const CUtensorMap &tx, const CUtensorMap &tw, const TcParams &tp, int P, cudaStream_t s) {
    switch (mt) {
        case 16: return launch_one<MODE, 16, 8>(tx, tw, tp, P, s);
        case 32: return launch_one<MODE, 32, 8>(tx, tw, tp, P, s);
        case 64: return launch_one<MODE, 64, 8>(tx, tw, tp, P, s);
        case 128: return launch_one<MODE, 128, 6>(tx, tw, tp, P, s);
        case 256: return launch_one<MODE, 256, 4>(tx, tw, tp, P, s);
    }
    return cudaErrorInvalidValue;
}

// Weight-only matmuls with few rows go to the persistent stream-K kernel with fused dequant
// (wq_tc.cu); with many rows to the expand-then-dense path (dequant.cu).  B200_QMM_WQ_DENSE_M sets
// the switch point.
int wq_dense_threshold(const MatmulArgs &p) {
    if (const char *e = getenv("B200_QMM_WQ_DENSE_M")) return atoi(e);
    // Group-wise int4 under bf16 activations with the fp16-product form switched off keeps the exact per-group fold in the
    // streaming kernel (its pre-scaled mode would round the weights to bf16), which falls behind expansion above 64 rows.
    if (p.a_type == ET_BF16 && p.b_type == ET_I4 && p.group < p.K) {
        const char *v = getenv("B200_QMM_WQ_BF16_VIA_F16");
        if (v && atoi(v) == 0) return 64;
    }
    return 128;
}
bool is_wq(const MatmulArgs &p) { return p.epilogue == EPI_PLAIN && p.scale && !p.a_scale && !p.b_scale; }
bool is_mx(const MatmulArgs &p) { return p.epilogue == EPI_PLAIN && p.a_scale && p.b_scale; }
bool use_stream_wq(const MatmulArgs &p) {
    return is_wq(p) && wq_tc_supported(p) && (p.M <= wq_dense_threshold(p) || !expand_supported(p));
}
// MX matmuls whose shape the native block-scaled kernel takes (mx_tc.cu); the others are expanded to bf16.
bool use_mx_native(const MatmulArgs &p) { return is_mx(p) && mx_native_supported(p); }
bool use_expand(const MatmulArgs &p) { return (is_mx(p) || is_wq(p)) && !use_stream_wq(p) && !use_mx_native(p) && expand_supported(p); }
// Decode shapes of int4 weights: register-dequant kernel (wq_mma.cu).
bool use_decode_wq(const MatmulArgs &p) { return use_stream_wq(p) && wq_mma_supported(p); }

}  // namespace

bool dense_tc_supported(const MatmulArgs &p) {
    if (dev_info().sm100 != 1 || !encode_fn()) return false;
    if (p.batch != 1 || p.b_transposed || p.accumulate || p.M < 1) return false;
    if (p.M > (1 << 24) || p.N > (1 << 24) || p.K > (1 << 24)) return false;
    if (p.epilogue == EPI_DEQ_I32 || p.epilogue == EPI_RAW_I32) {
        if (p.a_type != ET_I8 || p.b_type != ET_I8) return false;
        return p.K % 16 == 0 && p.N % 16 == 0;
    }
    if (p.epilogue == EPI_PLAIN && !p.scale && !p.a_scale && !p.b_scale) {
        if (p.a_type != p.b_type || (p.a_type != ET_BF16 && p.a_type != ET_F16)) return false;
        return p.K % 8 == 0 && p.N % 8 == 0;
    }
    return false;
}

uint64_t dense_tc_workspace_bytes(const MatmulArgs &p) { return make_plan(p).partial_bytes; }

cudaError_t launch_dense_tc(const MatmulArgs &p, cudaStream_t s) {
    const TcPlan pl = make_plan(p);
    if (p.workspace_bytes < pl.partial_bytes) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15)) return cudaErrorMisalignedAddress;
    if (pl.rowtile && (reinterpret_cast<uintptr_t>(p.out) & 15)) return cudaErrorMisalignedAddress;

    CUtensorMap tx, tw;
    bool ok;
    // With one row tile every weight byte is read once by one CTA: asking L2 for wider lines than the
    // box needs only slows the stream (measured on the decode kernel).  With several row tiles the
    // CTAs that share a weight tile run together and the wider fetch is kept.
    const CUtensorMapL2promotion w_promo = pl.m_tiles == 1 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    if (pl.mode == D_I8) {
        ok = make_map(&tx, p.a, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.K, p.M, p.K, 128, pl.mt, CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_map(&tw, p.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.N, p.K, p.N, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B, w_promo);
    } else {
        const CUtensorMapDataType dt = pl.mode == D_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        ok = make_map(&tx, p.a, dt, p.K, p.M, p.K * 2, 64, pl.mt, CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_map(&tw, p.b, dt, p.N, p.K, p.N * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B, w_promo);
    }
    if (!ok) return cudaErrorInvalidValue;

    TcParams tp{};
    tp.out = p.out;
    tp.partial = pl.split > 1 ? p.workspace : nullptr;
    tp.scale = p.scale; tp.bias = p.bias; tp.pertoken = p.pertoken;
    tp.sc_type = p.sc_type; tp.bias_type = p.bias_type; tp.out_type = p.out_type; tp.epilogue = p.epilogue;
    tp.M = (int)p.M; tp.N = (int)p.N; tp.K = (int)p.K;
    tp.m_tiles = pl.m_tiles; tp.tiles = pl.tiles; tp.num_kb = pl.num_kb; tp.kb_per_split = pl.kb_per_split; tp.units = pl.units;
    tp.full_units = pl.full_units; tp.tail_tiles = pl.tail_tiles; tp.split = pl.split; tp.mt = pl.mt; tp.tn = pl.tn;

    cudaError_t e;
    if (pl.rowtile) {
        switch (pl.mode) {
            case D_I8: e = launch_rowtile<D_I8>(tx, tw, tp, pl.P, s); break;
            case D_BF16: e = launch_rowtile<D_BF16>(tx, tw, tp, pl.P, s); break;
            default: e = launch_rowtile<D_F16>(tx, tw, tp, pl.P, s); break;
        }
    } else
    switch (pl.mode) {
        case D_I8: e = dispatch_mt<D_I8>(pl.mt, tx, tw, tp, pl.P, s); break;
        case D_BF16: e = dispatch_mt<D_BF16>(pl.mt, tx, tw, tp, pl.P, s); break;
        default: e = dispatch_mt<D_F16>(pl.mt, tx, tw, tp, pl.P, s); break;
    }
    if (e != cudaSuccess) return e;
    if (pl.split > 1) {
        const size_t elems = (size_t)pl.tail_tiles * pl.mt * pl.tn;
        tc_finalize_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, s>>>(tp);
        count_launch();
        e = cudaGetLastError();
    }
    return e;
}

// ---- dispatch of the tensor-core family ----------------------------------------------------------
// int4 weights in the tile-packed layout are read directly by the decode kernel (M <= 16).  Every other
// kernel reads the caller's [K,N] layout, so for them the weights are first laid back into that layout at
// the head of the workspace (one pass over the packed bytes) and the call proceeds as usual.
namespace {
inline uint64_t nz_copy_bytes(const MatmulArgs &p) { return align_up_u64((uint64_t)p.K * p.N / 2, 256); }
inline bool nz_direct(const MatmulArgs &p) { return p.b_nz && is_wq(p) && wq_mma_supported(p); }
inline MatmulArgs as_nd(const MatmulArgs &p, const void *w_nd) {
    MatmulArgs q = p;
    q.b_nz = false;
    if (w_nd) q.b = w_nd;
    return q;
}
}  // namespace

bool tc_supported(const MatmulArgs &p) {
    if (dev_info().sm100 != 1 || !encode_fn()) return false;
    if (p.b_nz && is_mx(p)) return mx_native_supported(p);   // fp4 weights widened at load time: the native kernel only
    if (p.b_nz) {
        if (!is_wq(p) || p.b_type != ET_I4) return false;
        return nz_direct(p) || (p.N % 8 == 0 && tc_supported(as_nd(p, nullptr)));
    }
    if (use_stream_wq(p) || use_expand(p) || use_mx_native(p)) return true;
    return dense_tc_supported(p);
}

void tc_plan(MatmulArgs &p) {
    if (p.b_nz) { p.split_k = 1; return; }   // either on-device weight format: no K split
    p.split_k = (use_stream_wq(p) || use_expand(p) || use_mx_native(p)) ? 1 : make_plan(p).split;
}

uint64_t tc_workspace_bytes(const MatmulArgs &p) {
    if (p.b_nz && is_mx(p)) return mx_native_workspace_bytes(p);
    if (p.b_nz) return nz_direct(p) ? wq_mma_workspace_bytes(p) : nz_copy_bytes(p) + tc_workspace_bytes(as_nd(p, nullptr));
    if (use_decode_wq(p)) return wq_mma_workspace_bytes(p);
    if (use_stream_wq(p)) return wq_tc_workspace_bytes(p);
    if (use_mx_native(p)) return mx_native_workspace_bytes(p);
    if (use_expand(p)) return expand_workspace_bytes(p);
    return dense_tc_workspace_bytes(p);
}

cudaError_t launch_tc(const MatmulArgs &p, cudaStream_t s) {
    if (p.b_nz && is_mx(p)) return launch_mx_native(p, s);
    if (p.b_nz) {
        if (nz_direct(p)) return launch_wq_mma(p, s);
        const uint64_t copy = nz_copy_bytes(p);
        if (!p.workspace || p.workspace_bytes < copy) return cudaErrorInvalidValue;
        if ((reinterpret_cast<uintptr_t>(p.b) & 15) || (reinterpret_cast<uintptr_t>(p.workspace) & 15)) return cudaErrorMisalignedAddress;
        cudaError_t e = launch_wq_unpack_nz(p.b, p.workspace, p.K, p.N, s);
        if (e != cudaSuccess) return e;
        MatmulArgs q = as_nd(p, p.workspace);
        q.workspace = (char *)p.workspace + copy;
        q.workspace_bytes = p.workspace_bytes - copy;
        return launch_tc(q, s);
    }
    if (use_decode_wq(p)) return launch_wq_mma(p, s);
    if (use_stream_wq(p)) return launch_wq_tc(p, s);
    if (use_mx_native(p)) return launch_mx_native(p, s);
    if (use_expand(p)) return launch_expand(p, s);
    return launch_dense_tc(p, s);
}

void tc_reserve_sms(int n) { g_reserved_sms = n > 0 ? n : 0; }

void tc_device_status_reset() {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(z));
    wq_tc_device_status_reset();
    wq_mma_device_status_reset();
    mx_tc_device_status_reset();
    wq_rows_device_status_reset();
    dynquant_device_status_reset();
}

unsigned int tc_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    const unsigned int w = wq_tc_device_status(), d = wq_mma_device_status(), x = mx_tc_device_status();
    const unsigned int r = wq_rows_device_status(), a = dynquant_device_status();
    return v ? v : (w ? w : (d ? d : (x ? x : (r ? r : a))));
}

}  // namespace qmm
