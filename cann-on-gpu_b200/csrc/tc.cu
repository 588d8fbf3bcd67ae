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
    int mt;                   // rows per tile (for the finalize kernel)
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
                            store_from_float(p.out, p.out_type, o, __uint_as_float(v[j]) + bf);
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

// Split-K reduction + epilogue: out = epi(sum_z partial[z]).
__global__ void tc_finalize_kernel(TcParams p) {
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x, per_tile = (size_t)p.mt * TILE_N;
    if (e >= per_tile * p.tail_tiles) return;
    const int t = (int)(e / per_tile), ml = (int)((e / TILE_N) % p.mt), nl = (int)(e % TILE_N);
    const int tile = p.full_units + t;
    const int n = (tile / p.m_tiles) * TILE_N + nl, m = (tile % p.m_tiles) * p.mt + ml;
    if (n >= p.N || m >= p.M) return;
    const size_t i = (size_t)m * p.N + n, stride = per_tile * p.tail_tiles, off = e;
    if (p.epilogue == EPI_PLAIN) {
        float v = 0.f;
        for (int z = 0; z < p.split; ++z) v += ((const float *)p.partial)[z * stride + off];
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
    int mode, mt, bk, split, num_kb, kb_per_split, m_tiles, tiles, units, P, full_units, tail_tiles;
    uint64_t partial_bytes;
};

TcPlan make_plan(const MatmulArgs &p) {
    TcPlan pl{};
    pl.mode = p.a_type == ET_I8 ? D_I8 : (p.a_type == ET_BF16 ? D_BF16 : D_F16);
    pl.bk = pl.mode == D_I8 ? 128 : 64;
    pl.mt = 16;
    while (pl.mt < p.M && pl.mt < 256) pl.mt *= 2;
    pl.num_kb = (int)((p.K + pl.bk - 1) / pl.bk);
    const int n_tiles = (int)((p.N + TILE_N - 1) / TILE_N);
    pl.m_tiles = (int)((p.M + pl.mt - 1) / pl.mt);
    pl.tiles = n_tiles * pl.m_tiles;
    const int sms = dev_info().sms > 0 ? dev_info().sms : 148;
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
            double t = rounds * kbps * pl.bk * (pl.mt + TILE_N) * elem / 45e9;
            if (eff > 1) t += 2.0 * eff * (double)pl.tail_tiles * pl.mt * TILE_N * 4.0 / 3e12 + 3e-6;
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
    pl.partial_bytes = pl.split > 1 ? (uint64_t)pl.split * pl.tail_tiles * pl.mt * TILE_N * 4 : 0;
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
int wq_dense_threshold() {
    const char *e = getenv("B200_QMM_WQ_DENSE_M");
    return e ? atoi(e) : 128;
}
bool is_wq(const MatmulArgs &p) { return p.epilogue == EPI_PLAIN && p.scale && !p.a_scale && !p.b_scale; }
bool is_mx(const MatmulArgs &p) { return p.epilogue == EPI_PLAIN && p.a_scale && p.b_scale; }
bool use_stream_wq(const MatmulArgs &p) {
    return is_wq(p) && wq_tc_supported(p) && (p.M <= wq_dense_threshold() || !expand_supported(p));
}
bool use_expand(const MatmulArgs &p) { return (is_mx(p) || is_wq(p)) && !use_stream_wq(p) && expand_supported(p); }
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
    tp.full_units = pl.full_units; tp.tail_tiles = pl.tail_tiles; tp.split = pl.split; tp.mt = pl.mt;

    cudaError_t e;
    switch (pl.mode) {
        case D_I8: e = dispatch_mt<D_I8>(pl.mt, tx, tw, tp, pl.P, s); break;
        case D_BF16: e = dispatch_mt<D_BF16>(pl.mt, tx, tw, tp, pl.P, s); break;
        default: e = dispatch_mt<D_F16>(pl.mt, tx, tw, tp, pl.P, s); break;
    }
    if (e != cudaSuccess) return e;
    if (pl.split > 1) {
        const size_t elems = (size_t)pl.tail_tiles * pl.mt * TILE_N;
        tc_finalize_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, s>>>(tp);
        count_launch();
        e = cudaGetLastError();
    }
    return e;
}

// ---- dispatch of the tensor-core family ----------------------------------------------------------
bool tc_supported(const MatmulArgs &p) {
    if (dev_info().sm100 != 1 || !encode_fn()) return false;
    if (use_stream_wq(p) || use_expand(p)) return true;
    return dense_tc_supported(p);
}

void tc_plan(MatmulArgs &p) { p.split_k = (use_stream_wq(p) || use_expand(p)) ? 1 : make_plan(p).split; }

uint64_t tc_workspace_bytes(const MatmulArgs &p) {
    if (use_decode_wq(p)) return wq_mma_workspace_bytes(p);
    if (use_stream_wq(p)) return wq_tc_workspace_bytes(p);
    if (use_expand(p)) return expand_workspace_bytes(p);
    return dense_tc_workspace_bytes(p);
}

cudaError_t launch_tc(const MatmulArgs &p, cudaStream_t s) {
    if (use_decode_wq(p)) return launch_wq_mma(p, s);
    if (use_stream_wq(p)) return launch_wq_tc(p, s);
    if (use_expand(p)) return launch_expand(p, s);
    return launch_dense_tc(p, s);
}

unsigned int tc_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    const unsigned int w = wq_tc_device_status(), d = wq_mma_device_status();
    return v ? v : (w ? w : d);
}

}  // namespace qmm
