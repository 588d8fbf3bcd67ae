// W4A16 / W8A16 decode kernel (M <= 16): packed weights streamed by TMA, dequantised in registers,
// multiplied on the warp-level tensor-core path (mma.sync m16n8k16, fp16), scales folded in fp32,
// stream-K over (tile, 128-row stage) units.
//
// Why not tcgen05 here: at decode shapes the matmul is a stream of weights from HBM, and feeding the
// 5th-generation tensor core means writing every dequantised weight back to shared memory (2 B per
// 4-bit weight) and having the MMA read it again -- shared-memory traffic that costs more than the HBM
// stream itself.  Here a packed weight is read from shared memory once (0.5 B), expanded by one
// lop3 per pair of weights, and goes to the tensor core from registers.
//
// The product always runs in fp16.  A 4-bit integer is exact in fp16, and the 10-bit mantissa has
// room for a nibble at bits 0-3 and another at bits 4-7, so one 32-bit word of eight nibbles becomes four
// fp16x2 registers with four lop3 and one shift (bf16's 7-bit mantissa would need a shift per
// register).  bf16 activations are converted to fp16 per stage with a power-of-two scale per row, which
// is exact (8 significant bits into 11) for every element within 2^-29 of the row's largest in that
// stage; the fold multiplies the scale back in fp32.
//
// Per CTA (one per SM, 16 warps):
//   warp 0       weight producer: one copy per stage (128 K rows x 256 columns of packed int4 = 16 KB)
//                into a ring of 6-9 slots.  Weights in the caller's [K,N] layout come as a 2-D TMA box
//                (128 rows x 128 B, 128-byte swizzle, no L2 promotion); weights in the tile-packed
//                layout (see wq_pack_nz_kernel) as one contiguous 16 KB bulk copy.
//   warps 14-15  activation producers (alternate stages): each loads its stage's 128 K columns of every activation row from
//                global memory (L2), converts them to scaled fp16, and writes them into the slot in
//                B-fragment order together with the row's scale and the row's sum over the stage.
//   warps 1-12   three teams of four warps; a team owns every third stage, each of its warps 64 of the
//                tile's 256 columns.  Per 16 K rows a lane turns 32 nibbles into 16 fp16x2 A-fragment
//                registers holding the exact integers 1032 + q (even columns) and 1152 + 16 q (odd
//                columns); the activations are the B fragments.  At the end of the stage
//                    tot += s_g[n] * 2^e[m] * (acc - (1032 + off_g[n]) * sum_stage x[m])
//                which is the reference's algebra (cuda/src/ops/matmul.cu:334-335) per stage, in fp32.
//   warp 13      reducer: when all teams have finished a tile (or this CTA's piece of it) it sums the
//                teams' partial tiles from shared memory in a fixed order and writes the output
//                (whole tile) or an fp32 partial tile in the workspace (piece); the CTA that finds all pieces of a
//                tile published sums them and writes the tile, so one launch does everything.
// Work split: the (tile, stage) space is cut into gridDim.x equal contiguous shares (stream-K).
// The ring depth is a multiple of the team count, so every slot belongs to one team, which meets the
// phases of the slot's barrier in order: a parity wait is never asked about a phase that is two ahead.
//
// int8 weights use the same path: a byte is lo + 16 * hi (unsigned low nibble, signed high nibble); the
// two nibbles ride rows g and g+8 of one mma and are recombined in the fold (tile = 128 columns).
//
// Replaces the reference's k_wq_fused (cuda/src/ops/matmul.cu:337-352).
#include <atomic>
#include <chrono>
#include <cmath>
#include <mutex>
#include <type_traits>

#include "tc_common.cuh"

namespace qmm {
namespace {

constexpr int MM_TILE_N = 256;      // nibble columns per tile
constexpr int MM_SBK = 128;         // K rows per stage
constexpr int MM_W_BYTES = 16384;   // packed weights of one stage: 128 rows x 128 B
constexpr int MM_TEAMS = 3;
constexpr int MM_MAX_ROWS = 16;     // rows of one pass (two activation fragments of 8)
constexpr int MM_XP = 2;            // activation producer warps (they take alternate stages)
constexpr int MM_MAX_PEERS = 8;     // GPUs of a gathering epilogue
constexpr int MM_THREADS = (4 * MM_TEAMS + 2 + MM_XP) * 32;

struct MmParams {
    void *out;
    float *slots;            // [tiles + P][M][tile_n] fp32 partial tiles of tiles shared between CTAs
    unsigned long long *tags;   // [tiles] per tile: this launch's key | number of partial tiles published
    unsigned long long nonce;   // this launch's key: upper 48 bits, never 0; the lower 16 are zero
    const void *x;           // activations [M,K], bf16 or fp16
    const void *scale, *offset, *bias;
    const uint8_t *wnz;      // tile-packed weights (blocks of 16 KB, [tile][stage]) or null
    const uint8_t *xf;       // nine to sixteen rows: the activations converted per stage by wq_mma_activation_kernel
    int x_bf16;              // activation / scale / output type: 1 = bf16, 0 = fp16
    int M, N, K;
    int num_sb;              // stages per tile = ceil(K / 128)
    long long total_u;       // tiles * num_sb
    int gsb;                 // stages per scale row (num_sb for per-channel scales)
    int ns;                  // ring slots (a multiple of the team count)
    int tile_n;              // output columns per tile: 256 (int4) or 128 (int8: two nibbles per column)
    int weights_early;       // weights, scales and offsets may be read before the preceding kernel has completed
    unsigned long long wait_ns;   // time limit of every wait (0 = about a second)
    int test_drop;           // test hook: CTA 0 never fetches its first stage, so the wait for it runs out
    // Gathering epilogue (column shards over several GPUs): besides p.out every finished output row is stored into each
    // peer's receive window as 8-byte packets {two 16-bit outputs, the call's number}; the receiver polls the numbers.
    int gather_n, gather_rank;                    // GPUs taking part (0 = no gathering), this GPU's index
    int gather_f32;                               // packets {one fp32 output, number} to every GPU, this one included (partial
                                                  // results that the receiver sums), instead of {two 16-bit outputs, number}
    unsigned long long gather_peer[MM_MAX_PEERS]; // every GPU's window as this process sees it
    unsigned long long gather_buf_bytes;          // one of the window's two receive buffers (they alternate by call)
    const unsigned long long *gather_calls;       // calls completed so far (device memory, advanced by the receiver)
};

// Shared memory of one CTA: [ring: ns slots][partial tiles: teams x M rows x 256 fp32][barriers][flag].
// A slot: [packed weights 16 KB][activations in B-fragment order, MF x 2 KB][row scales 16 f32][row sums 16 f32]
// [the stage's scale row for the tile's columns, 512 B][its offset row, 512 B].
template <int MF>
struct MmSmem {
    static constexpr int XF_OFF = MM_W_BYTES;
    static constexpr int META_OFF = XF_OFF + MF * 2048;
    static constexpr int SC_OFF = META_OFF + 128;
    static constexpr int OF_OFF = SC_OFF + 512;
    static constexpr int SLOT = (OF_OFF + 512 + 1023) / 1024 * 1024;
    __host__ __device__ static int part_bytes(int M) { return MM_TEAMS * M * MM_TILE_N * 4; }   // sized for the wider (int4) tile
    __host__ __device__ static int bar_off(int ns, int M) { return ns * SLOT + part_bytes(M); }
    __host__ __device__ static int total(int ns, int M) { return bar_off(ns, M) + (2 * ns + 2) * 8 + 16 + 1024; }
};

#ifdef WQ_MMA_PROFILE
// Time stamps per CTA (development aid, compiled only with -DWQ_MMA_PROFILE): row 0 entry, 1 barriers initialised,
// 2 weight producer past its dependency wait, 3 first stage full, 4 last stage multiplied (latest team), 5 reducer
// has the teams' last partial tile, 6 reducer done, 7 nanoseconds the reducer spent on tiles shared between CTAs.
__device__ unsigned long long g_mm_prof[8][160];
#define MM_STAMP(row) do { g_mm_prof[row][blockIdx.x < 160 ? blockIdx.x : 159] = global_ns(); } while (0)
#define MM_STAMP_MAX(row) do { atomicMax(&g_mm_prof[row][blockIdx.x < 160 ? blockIdx.x : 159], global_ns()); } while (0)
#else
#define MM_STAMP(row) do { } while (0)
#define MM_STAMP_MAX(row) do { } while (0)
#endif

// The (tile, stage) space is cut into one contiguous share per CTA: CTA c works on units [b[c], b[c + 1]).
constexpr int MM_MAX_CTAS = 256;
struct MmShares { long long b[MM_MAX_CTAS + 1]; };

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same with a zero C operand: the first step of a stage needs no cleared accumulators.
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Two nibbles of a word -> two fp16 holding integers above a power of two: (v & mask) ^ magic in one
// lop3, both constants in registers.  mask 0x000F000F, magic 0x6408: 1024 + (nibble ^ 8) = 1032 + q for a
// two's-complement nibble q; mask 0x00F000F0, magic 0x6480: 1024 + 16 * (nibble ^ 8) = 1152 + 16 q.
__device__ __forceinline__ uint32_t dq_pair(uint32_t v, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(v), "r"(mask), "r"(magic));
    return r;
}
// 16-byte read-only load, issued where it is written (the compiler may not sink it to its use).
__device__ __forceinline__ uint4 ldg16_now(const void *ptr) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}
__device__ __forceinline__ uint2 ldg8_now(const void *ptr) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
    return v;
}
template <bool BF16> __device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    if constexpr (BF16) return __uint_as_float(h << 16);
    return __half2float(__ushort_as_half((unsigned short)h));
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Programmatic dependent launch: with the launch attribute set, a CTA of this kernel may start on an SM as
// soon as the kernel before it in the stream has let go of that SM (instead of after the whole grid has
// drained), so its start-up -- barrier initialisation, clearing shared memory -- overlaps the predecessor's
// tail.  Nothing of this kernel touches global memory before pdl_wait_for_prerequisites(), which returns once the
// predecessor has completed and its writes are visible; without the attribute both calls do nothing.
__device__ __forceinline__ void pdl_wait_for_prerequisites() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The bounded wait of this kernel: like mbar_wait, with the time limit a launch parameter (0 = the common limit of
// about a second) so that a test can make every wait run out at once and see the kernel come back with a status.
__device__ __forceinline__ bool mm_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned code, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns(), limit = limit_ns ? limit_ns : WAIT_LIMIT_NS;
    unsigned it = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++it & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(&g_tc_status, 0u, code);
                return false;
            }
        }
    }
}

// Bounded wait that ignores the abort flag (used only to let copies in flight land before exit).
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (global_ns() - t0 > 2000000ull) return;
    }
}

// EPL consecutive elements of one activation row (V = EPL / 4 packed 8-byte words per lane; 128 / EPL lanes share
// the row) -> scaled fp16 pairs h, the row's scale 2^e (up) and the row's sum of the converted values.
template <bool BF16, int EPL>
__device__ __forceinline__ void mm_convert_rows(const uint2 (&cur)[EPL / 4], uint32_t (&h)[EPL / 2], float &up, float &sum) {
    constexpr int LPR = 128 / EPL, V = EPL / 4;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const uint32_t w[2] = {cur[j].x, cur[j].y};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            if constexpr (BF16) {
                v[4 * j + 2 * c] = __uint_as_float(w[c] << 16);
                v[4 * j + 2 * c + 1] = __uint_as_float(w[c] & 0xFFFF0000u);
            } else {
                const float2 h2 = __half22float2(*reinterpret_cast<const __half2 *>(&w[c]));
                v[4 * j + 2 * c] = h2.x;
                v[4 * j + 2 * c + 1] = h2.y;
            }
        }
    }
    float down = 1.f;
    up = 1.f;
    if constexpr (BF16) {
        // the largest magnitude of the row: bf16 magnitudes order like their 15-bit patterns, two per word
        uint32_t mx2 = 0u;
#pragma unroll
        for (int j = 0; j < V; ++j) mx2 = __vmaxu2(mx2, __vmaxu2(cur[j].x & 0x7FFF7FFFu, cur[j].y & 0x7FFF7FFFu));
        uint32_t abits = max(mx2 & 0xFFFFu, mx2 >> 16) << 16;
        if constexpr (LPR == 32) abits = __reduce_max_sync(0xffffffffu, abits);
        else {
#pragma unroll
            for (int o = 1; o < LPR; o <<= 1) abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, o));
        }
        // it lands in [2^14, 2^15); zero rows keep scale 1; an infinite (or NaN) row is clamped (its result is not
        // finite either way)
        int e = 0;
        if (abits != 0u) {
            e = (int)((abits >> 23) & 0xFFu) - 127 - 14;
            e = e < -100 ? -100 : (e > 100 ? 100 : e);
        }
        down = __uint_as_float((uint32_t)(127 - e) << 23);
        up = __uint_as_float((uint32_t)(127 + e) << 23);
    }
    float sm = 0.f;
#pragma unroll
    for (int c = 0; c < EPL / 2; ++c) {
        h[c] = pack_f16x2(v[2 * c] * down, v[2 * c + 1] * down);
        const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&h[c]));
        sm += back.x + back.y;   // the sum of what the tensor core will see
    }
#pragma unroll
    for (int o = 1; o < LPR; o <<= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
    sum = sm;
}
// Writes them in B-fragment order (step st of 16 K, lane (g = row, t): {k = 2t, 2t+1}, {k = 2t+8, 2t+9}) behind `xf`,
// followed by the 16 row scales and the 16 row sums (the layout of a slot's activation region).
template <int MF, int EPL>
__device__ __forceinline__ void mm_store_rows(uint8_t *xf, int f, int lane, const uint32_t (&h)[EPL / 2], float up, float sum) {
    constexpr int LPR = 128 / EPL;
    const int q = lane % LPR, rsub = lane / LPR;
#pragma unroll
    for (int c = 0; c < EPL / 2; ++c) {
        const int kk = EPL * q + 2 * c, st = kk >> 4, kr = kk & 15;
        *reinterpret_cast<uint32_t *>(xf + f * 2048 + (((st * 32 + 4 * rsub + ((kr & 7) >> 1)) << 3) + 4 * (kr >> 3))) = h[c];
    }
    if (q == 0) {
        const int row = (MF == 2 ? 8 * f : 0) + rsub;
        *reinterpret_cast<float *>(xf + MF * 2048 + 4 * row) = up;
        *reinterpret_cast<float *>(xf + MF * 2048 + 64 + 4 * row) = sum;
    }
}

// Five to sixteen rows: converting that many rows per stage in every CTA is more than two warps can keep up with (they
// share their schedulers with the compute warps), and it is the same work in all CTAs (the activations do not depend on
// the tile).  One small kernel converts each 128-column stage of the activations once into the layout of a slot's
// activation region; the main kernel then copies that region with the weights.
template <bool BF16, int MF>
__global__ void __launch_bounds__(32) wq_mma_activation_kernel(const uint16_t *x, uint8_t *xf_all, int M, int K) {
    pdl_launch_dependents();
    const int sbi = blockIdx.x, lane = threadIdx.x;
    constexpr int EPL = 32, V = EPL / 4, LPR = 128 / EPL;
    const int q = lane % LPR, rsub = lane / LPR, k = sbi * MM_SBK + EPL * q;
    uint8_t *xf = xf_all + (size_t)sbi * (MF * 2048 + 128);
#pragma unroll
    for (int f = 0; f < MF; ++f) {
        const int m = 8 * f + rsub;
        uint2 cur[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            cur[j] = make_uint2(0u, 0u);
            if (m < M && k + 4 * j < K) cur[j] = ldg8_now(x + (size_t)m * K + k + 4 * j);
        }
        uint32_t h[EPL / 2];
        float up, sum;
        mm_convert_rows<BF16, EPL>(cur, h, up, sum);
        mm_store_rows<MF, EPL>(xf, f, lane, h, up, sum);
    }
}

// The activation producer (one warp).  For every stage of the CTA's share, in order: the stage's 128 K
// columns of every activation row, from global memory (L2) to scaled fp16 in the slot, in B-fragment order
// (step st of 16 K, lane (g = row, t): {k = 2t, 2t+1}, {k = 2t+8, 2t+9}), plus the row's scale 2^e and the
// row's sum over the stage.  A lane owns EPL consecutive elements of one row, so 128 / EPL lanes share a row
// and 32 / (128 / EPL) rows are handled per pass: EPL = 4 serves one row with all 32 lanes, 32 serves eight
// rows (two passes for nine to sixteen).  Rows the passes never touch stay zero from the kernel's start.
// Loads run D stages ahead of the conversion so that the L2 round trip is not paid per stage.
template <bool BF16, int MF, int EPL>
__device__ __forceinline__ void mm_activation_producer(const MmParams &p, uint32_t base, int NS, uint32_t bars, volatile int *abort_flag,
                                                       int sb0, int nu, int lane, int xp) {
    using L = MmSmem<MF>;
    constexpr int LPR = 128 / EPL, R = 32 / LPR, V = EPL / 4, D = EPL <= 8 ? 4 : 2;
    const int q = lane % LPR, rsub = lane / LPR;
    const uint16_t *xg = static_cast<const uint16_t *>(p.x);
    uint2 buf[D][MF][V];
    auto load_stage = [&](int sbi, uint2 (&v)[MF][V]) {
        const int k = sbi * MM_SBK + EPL * q;
#pragma unroll
        for (int f = 0; f < MF; ++f) {
            const int m = (MF == 2 ? 8 * f : 0) + rsub;
#pragma unroll
            for (int j = 0; j < V; ++j) {
                v[f][j] = make_uint2(0u, 0u);
                if (m < p.M && k + 4 * j < p.K) v[f][j] = ldg8_now(xg + (size_t)m * p.K + k + 4 * j);   // K % 8 == 0
            }
        }
    };
    auto next_sb = [&](int sbi, int by) { int s2 = sbi + by; while (s2 >= p.num_sb) s2 -= p.num_sb; return s2; };
    pdl_wait_for_prerequisites();   // the activations are the predecessor's output
    // this warp's stages are xp, xp + MM_XP, ... of the share
    int sb_load = next_sb(sb0, xp % p.num_sb);
#pragma unroll
    for (int d = 0; d < D; ++d) {
        if (xp + MM_XP * d < nu) load_stage(sb_load, buf[d]);
        sb_load = next_sb(sb_load, MM_XP % p.num_sb);
    }
    int slot = xp % NS, round = xp / NS;
    for (int i0 = xp; i0 < nu; i0 += MM_XP * D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const int i = i0 + MM_XP * d;
            if (i >= nu) break;
            uint2 cur[MF][V];
#pragma unroll
            for (int f = 0; f < MF; ++f)
#pragma unroll
                for (int j = 0; j < V; ++j) cur[f][j] = buf[d][f][j];
            if (i + MM_XP * D < nu) load_stage(sb_load, buf[d]);
            sb_load = next_sb(sb_load, MM_XP % p.num_sb);
            // convert first (registers only), then wait for the slot: what remains after the wait is a few stores
            uint32_t h[MF][EPL / 2];
            float up[MF], sum[MF];
#pragma unroll
            for (int f = 0; f < MF; ++f) mm_convert_rows<BF16, EPL>(cur[f], h[f], up[f], sum[f]);
            if (round > 0 && !mm_wait(bars + 8u * (NS + slot), (round - 1) & 1, abort_flag, 0x340u + slot, p.wait_ns)) return;
            uint8_t *xf = static_cast<uint8_t *>(__cvta_shared_to_generic(base + slot * L::SLOT + L::XF_OFF));
#pragma unroll
            for (int f = 0; f < MF; ++f) mm_store_rows<MF, EPL>(xf, f, lane, h[f], up[f], sum[f]);
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8u * slot);
            slot += MM_XP;
            while (slot >= NS) { slot -= NS; ++round; }
        }
    }
}

template <bool Q8, bool BF16, int MF, bool NZ>
__global__ void __launch_bounds__(MM_THREADS, 1)
wq_mma_kernel(const __grid_constant__ CUtensorMap tm_w, const MmParams p, const __grid_constant__ MmShares shares) {
    using L = MmSmem<MF>;
    constexpr int TN = Q8 ? 128 : 256;   // output columns per tile (the tile is 256 nibble columns wide)
    const int NS = p.ns;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    const int bar_off = L::bar_off(NS, p.M);
    const uint32_t bars = base + bar_off;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (NS + s); };
    const uint32_t seg_done = bars + 8u * (2 * NS), seg_free = bars + 8u * (2 * NS + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + bar_off + (2 * NS + 2) * 8);
    float *part = reinterpret_cast<float *>(gen_base + NS * L::SLOT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int P = gridDim.x, cta = blockIdx.x;
    if (threadIdx.x == 0) MM_STAMP(0);
    const bool has_off = p.offset != nullptr;
    const long long ub = shares.b[cta], ue = shares.b[cta + 1];
    const int nu = (int)(ue - ub);
    const int tile_first = (int)(ub / p.num_sb), tile_last = (int)((ue - 1) / p.num_sb);

    // Start-up.  The weight producer (thread 0) initialises the barriers itself and goes straight on to issue its first
    // copies; it only announces itself at the CTA barrier (warp 0 arrives without waiting).  The other fifteen warps
    // meanwhile clear the activation regions (rows the activation producers never write, those beyond M, must read as
    // zero) and wait at the barrier, after which they see the initialised barriers.  The first stage is thereby on its
    // way about a microsecond earlier than with a barrier for all, and that is time on the call's critical path.
    // A stage is full when the weight copy has landed (producer's arrive + bytes) and the activation producer has
    // arrived; it is empty when the team's four warps have arrived.
    if (warp == 0) {
        if (lane == 0) {
            for (int sl = 0; sl < NS; ++sl) { mbar_init(full_bar(sl), 2); mbar_init(empty_bar(sl), 4); }
            mbar_init(seg_done, 4 * MM_TEAMS);
            mbar_init(seg_free, 1);
            *abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            __threadfence_block();
        }
        __syncwarp();
        asm volatile("bar.arrive 0, %0;" ::"r"(MM_THREADS) : "memory");
    } else {
        for (int i = threadIdx.x - 32; i < NS * (MF * 512 + 32); i += MM_THREADS - 32) {
            const int sl = i / (MF * 512 + 32), w = i % (MF * 512 + 32);
            *reinterpret_cast<uint32_t *>(gen_base + sl * L::SLOT + L::XF_OFF + 4 * w) = 0u;
        }
        asm volatile("bar.sync 0, %0;" ::"r"(MM_THREADS) : "memory");
    }
    if (threadIdx.x == 0) pdl_launch_dependents();   // the next kernel in the stream may take over SMs as they free up
    if (threadIdx.x == 32) MM_STAMP(1);

    if (warp == 0) {
        // ------------------------------------------------------------------ weight producer
        if (lane == 0) {
            if (!p.weights_early) pdl_wait_for_prerequisites();
            MM_STAMP(2);
            // Everything the loop needs is kept incrementally (this is one thread competing with fifteen warps for
            // issue slots: every instruction here is paid in full, per stage).
            int i = 0, slot = 0, round = 0;
            int tile = tile_first, sbi = (int)(ub - (long long)tile_first * p.num_sb);
            int gcnt = sbi % p.gsb;                                          // stages into the current scale group
            const uint16_t *sc_src = static_cast<const uint16_t *>(p.scale) + (size_t)(sbi / p.gsb) * p.N + (size_t)tile * TN;
            const ptrdiff_t of_delta = has_off ? static_cast<const uint16_t *>(p.offset) - static_cast<const uint16_t *>(p.scale) : 0;
            const uint8_t *w_src = NZ ? p.wnz + ((size_t)tile * p.num_sb + sbi) * MM_W_BYTES : nullptr;   // blocks are [tile][stage]
            uint32_t row_bytes = (uint32_t)min(TN, p.N - tile * TN) * 2u;
            uint32_t dst = base, fbar = bars, ebar = bars + 8u * NS;
            bool ok = true;
            for (; i < nu; ++i) {
                if (round > 0 && !mm_wait(ebar, (round - 1) & 1, abort_flag, 0x300u + slot, p.wait_ns)) { ok = false; break; }
                // the stage's scale (and offset) row for this tile's columns rides with the weights, so the
                // consumers never wait on a global load
                if (!(p.test_drop && cta == 0 && i == 0)) {   // test hook: CTA 0 never fetches its first stage
                    mbar_expect_tx(fbar, MM_W_BYTES + (has_off ? 2u : 1u) * row_bytes);
                    if constexpr (NZ) bulk_load_1d(dst, w_src, MM_W_BYTES, fbar);
                    else tma_load_2d(dst, &tm_w, fbar, tile * 128, sbi * MM_SBK);
                    bulk_load_1d(dst + L::SC_OFF, sc_src, row_bytes, fbar);
                    if (has_off) bulk_load_1d(dst + L::OF_OFF, sc_src + of_delta, row_bytes, fbar);
                }
                if constexpr (NZ) w_src += MM_W_BYTES;
                dst += L::SLOT; fbar += 8u; ebar += 8u;
                if (++slot == NS) { slot = 0; ++round; dst = base; fbar = bars; ebar = bars + 8u * NS; }
                if (++gcnt == p.gsb) { gcnt = 0; sc_src += p.N; }
                if (++sbi == p.num_sb) {
                    sbi = 0; gcnt = 0; ++tile;
                    sc_src = static_cast<const uint16_t *>(p.scale) + (size_t)tile * TN;
                    row_bytes = (uint32_t)min(TN, p.N - tile * TN) * 2u;
                }
            }
            // Let the copies of the last ring's worth of stages land before the CTA's shared memory goes away.  In a
            // normal run the consumers have seen all of them (this returns at once); after a wait gave up anywhere in
            // the CTA the consumers may be gone while copies are still in flight.
            (void)ok;
            for (int b = (i > NS ? i - NS : 0); b < i; ++b) mbar_drain(full_bar(b % NS), (b / NS) & 1);
        }
    } else if (warp >= 4 * MM_TEAMS + 2) {
        // ------------------------------------------------------------------ activation producers
        const int sb0 = (int)(ub - (long long)tile_first * p.num_sb), xp = warp - (4 * MM_TEAMS + 2);
        if (p.xf != nullptr) {
            // converted once per call by wq_mma_activation_kernel: one bulk copy per stage
            if (xp == 0 && lane == 0) {
                pdl_wait_for_prerequisites();
                constexpr uint32_t XB = MF * 2048 + 128;
                int slot = 0, round = 0, sbi = sb0;
                for (int i = 0; i < nu; ++i) {
                    if (round > 0 && !mm_wait(empty_bar(slot), (round - 1) & 1, abort_flag, 0x340u + slot, p.wait_ns)) break;
                    mbar_expect_tx(full_bar(slot), XB);
                    bulk_load_1d(base + slot * L::SLOT + L::XF_OFF, p.xf + (size_t)sbi * XB, XB, full_bar(slot));
                    if (++slot == NS) { slot = 0; ++round; }
                    if (++sbi == p.num_sb) sbi = 0;
                }
            }
        } else if constexpr (MF == 1) {
            if (p.M == 1) mm_activation_producer<BF16, 1, 4>(p, base, NS, bars, abort_flag, sb0, nu, lane, xp);
            else if (p.M == 2) mm_activation_producer<BF16, 1, 8>(p, base, NS, bars, abort_flag, sb0, nu, lane, xp);
            else if (p.M <= 4) mm_activation_producer<BF16, 1, 16>(p, base, NS, bars, abort_flag, sb0, nu, lane, xp);
            else mm_activation_producer<BF16, 1, 32>(p, base, NS, bars, abort_flag, sb0, nu, lane, xp);
        }
    } else if (warp <= 4 * MM_TEAMS) {
        // ------------------------------------------------------------------ compute
        const int cw = warp - 1, team = cw >> 2, wq = cw & 3;
        const int g = lane >> 2, t = lane & 3;
        // caller's layout: byte offsets inside a slot of the four weight words of step 0 (rows 2t, 2t+1,
        // 2t+8, 2t+9 of this lane's 8 columns, under the 128-byte swizzle); packed layout: one 16-byte vector
        uint32_t woff[4];
        {
            const int c16 = 2 * wq + (g >> 2), inb = 4 * (g & 3);
            const int rows[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
            for (int j = 0; j < 4; ++j) woff[j] = 128 * rows[j] + (((c16 ^ (rows[j] & 7)) << 4)) + inb;
            if constexpr (NZ) woff[0] = (uint32_t)(wq * 8 * 512 + lane * 16);
        }
        // int4: every nibble is a signed weight (xor 8 -> q + 8 above 1024).  int8: the byte is
        // q = lo + 16 * hi with lo the unsigned low nibble (no xor) and hi the signed high nibble.
        uint32_t m1 = 0x000F000Fu, g1 = Q8 ? 0x64006400u : 0x64086408u, m2 = 0x00F000F0u, g2 = 0x64806480u;
        asm volatile("" : "+r"(m1), "+r"(g1), "+r"(m2), "+r"(g2));   // keep the constants in registers
        // first of this lane's columns inside the tile: 8 nibble columns = 8 (int4) or 4 (int8) outputs
        const int n_lane = Q8 ? 32 * wq + 4 * g : 64 * wq + 8 * g;
        const uint32_t xf_lane = L::XF_OFF + lane * 8, meta_lane = L::META_OFF + 8 * t;

        float acc[MF][4][4], tot[MF][4][4];
        bool ok = true;
        int sg = 0;
        for (int tile = tile_first; tile <= tile_last && ok; ++tile, ++sg) {
            const long long t_lo = (long long)tile * p.num_sb, t_hi = t_lo + p.num_sb;
            const int j_lo = (int)((t_lo > ub ? t_lo : ub) - ub), j_hi = (int)((t_hi < ue ? t_hi : ue) - ub);
            const int n_glob = tile * TN + n_lane;
            const bool n_ok = n_glob < p.N;
            bool had = false;
#pragma unroll
            for (int f = 0; f < MF; ++f)
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int e = 0; e < 4; ++e) tot[f][r][e] = 0.f;
            const int j_first = j_lo + (team - j_lo % MM_TEAMS + MM_TEAMS) % MM_TEAMS;
            for (int j = j_first; j < j_hi && ok; j += MM_TEAMS) {
                had = true;
                const int slot = j % NS, round = j / NS;
                if (!mm_wait(full_bar(slot), round & 1, abort_flag, 0x310u + slot, p.wait_ns)) { ok = false; break; }
                if (warp == 1 && lane == 0 && sg == 0 && j == j_first) MM_STAMP(3);
                const uint32_t sb = base + slot * L::SLOT;
#pragma unroll
                for (int st = 0; st < 8; ++st) {
                    // caller's layout: lo[i] / hi[i] hold rows (2t, 2t+1) / (2t+8, 2t+9) side by side in their two
                    // halves, columns 4i .. 4i+3; packed layout: word r holds both row pairs of columns 2r, 2r+1
                    uint32_t wv[4];
                    if constexpr (NZ) {
                        const uint4 v = lds128(sb + woff[0] + st * 512);
                        wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
                    } else {
                        const uint32_t w0 = lds32(sb + woff[0] + st * 2048), w1 = lds32(sb + woff[1] + st * 2048);
                        const uint32_t w2 = lds32(sb + woff[2] + st * 2048), w3 = lds32(sb + woff[3] + st * 2048);
                        wv[0] = __byte_perm(w0, w1, 0x5410); wv[1] = __byte_perm(w0, w1, 0x7632);
                        wv[2] = __byte_perm(w2, w3, 0x5410); wv[3] = __byte_perm(w2, w3, 0x7632);
                    }
                    uint2 b[MF];
#pragma unroll
                    for (int f = 0; f < MF; ++f) b[f] = lds64(sb + xf_lane + f * 2048 + st * 256);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        // a0 / a2: column 2r (even: 1032 + q) at rows (2t, 2t+1) / (2t+8, 2t+9); a1 / a3: column 2r+1
                        // (odd: 1152 + 16 q, taken in place from bits 4-7)
                        uint32_t a0, a1, a2, a3;
                        if constexpr (NZ) {
                            const uint32_t hi = wv[r] >> 8;
                            a0 = dq_pair(wv[r], m1, g1);
                            a1 = dq_pair(wv[r], m2, g2);
                            a2 = dq_pair(hi, m1, g1);
                            a3 = dq_pair(hi, m2, g2);
                        } else {
                            const uint32_t l = (r & 1) ? wv[r >> 1] >> 8 : wv[r >> 1], h = (r & 1) ? wv[2 + (r >> 1)] >> 8 : wv[2 + (r >> 1)];
                            a0 = dq_pair(l, m1, g1);
                            a1 = dq_pair(l, m2, g2);
                            a2 = dq_pair(h, m1, g1);
                            a3 = dq_pair(h, m2, g2);
                        }
#pragma unroll
                        for (int f = 0; f < MF; ++f) {
                            if (st == 0) mma16816_first(acc[f][r], a0, a1, a2, a3, b[f].x, b[f].y);
                            else mma16816(acc[f][r], a0, a1, a2, a3, b[f].x, b[f].y);
                        }
                    }
                }
                // row scales 2^e and row sums of this lane's two activation rows (m = 8 f + 2 t, + 1)
                float2 xsc[MF], xs[MF];
#pragma unroll
                for (int f = 0; f < MF; ++f) {
                    xsc[f] = lds64f(sb + meta_lane + 32 * f);
                    xs[f] = lds64f(sb + meta_lane + 64 + 32 * f);
                }
                // this lane's 8 columns of the stage's scale / offset row (4 columns for int8 weights)
                uint4 sraw = make_uint4(0, 0, 0, 0), oraw = sraw;
                if constexpr (Q8) {
                    const uint2 a = lds64(sb + L::SC_OFF + 2 * n_lane);
                    sraw.x = a.x; sraw.y = a.y;
                    if (has_off) { const uint2 c = lds64(sb + L::OF_OFF + 2 * n_lane); oraw.x = c.x; oraw.y = c.y; }
                } else {
                    sraw = lds128(sb + L::SC_OFF + 2 * n_lane);
                    if (has_off) oraw = lds128(sb + L::OF_OFF + 2 * n_lane);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(slot));
                // fold the finished stage (one uniform branch on the presence of offsets, so that the
                // common offset-free form carries no conversions or selects for them)
                const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w}, ow[4] = {oraw.x, oraw.y, oraw.z, oraw.w};
                auto fold = [&](auto off_tag) {
                    constexpr bool OFF = decltype(off_tag)::value;
                    if constexpr (Q8) {
                        // column r of this lane: rows g (low nibbles, 1024 + lo) and g+8 (high nibbles, 1152 + 16 hi)
                        // of the same mma
                        constexpr float C = 1024.f + 1152.f;
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const float sn = half_bits_to_float<BF16>((r & 1) ? sw[r >> 1] >> 16 : sw[r >> 1] & 0xFFFFu);
                            float cn = C;
                            if constexpr (OFF) cn += half_bits_to_float<BF16>((r & 1) ? ow[r >> 1] >> 16 : ow[r >> 1] & 0xFFFFu);
#pragma unroll
                            for (int f = 0; f < MF; ++f) {
                                tot[f][r][0] = fmaf(sn * xsc[f].x, fmaf(-cn, xs[f].x, acc[f][r][2] + acc[f][r][0]), tot[f][r][0]);
                                tot[f][r][1] = fmaf(sn * xsc[f].y, fmaf(-cn, xs[f].y, acc[f][r][3] + acc[f][r][1]), tot[f][r][1]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                // column 2r + h; odd columns were accumulated as 1152 + 16 q
                                float sn = half_bits_to_float<BF16>(h ? sw[r] >> 16 : sw[r] & 0xFFFFu);
                                float cn = h ? 1152.f : 1032.f;
                                if constexpr (OFF) {
                                    const float off = half_bits_to_float<BF16>(h ? ow[r] >> 16 : ow[r] & 0xFFFFu);
                                    cn += h ? 16.f * off : off;
                                }
                                if (h) sn *= 0.0625f;
#pragma unroll
                                for (int f = 0; f < MF; ++f) {
                                    tot[f][r][2 * h] = fmaf(sn * xsc[f].x, fmaf(-cn, xs[f].x, acc[f][r][2 * h]), tot[f][r][2 * h]);
                                    tot[f][r][2 * h + 1] = fmaf(sn * xsc[f].y, fmaf(-cn, xs[f].y, acc[f][r][2 * h + 1]), tot[f][r][2 * h + 1]);
                                }
                            }
                        }
                    }
                };
                if (has_off) fold(std::true_type{});
                else fold(std::false_type{});
            }
            if (!ok) break;
            if (wq == 0 && lane == 0 && tile == tile_last) MM_STAMP_MAX(4);
            // hand this team's partial tile to the reducer
            if (sg >= 1 && !mm_wait(seg_free, (sg - 1) & 1, abort_flag, 0x320u, p.wait_ns)) { ok = false; break; }
            if (had) {
#pragma unroll
                for (int f = 0; f < MF; ++f)
#pragma unroll
                    for (int r = 0; r < 4; ++r)
#pragma unroll
                        for (int e = 0; e < (Q8 ? 2 : 4); ++e) {
                            const int m = 8 * f + 2 * t + (e & 1), n = Q8 ? n_lane + r : n_lane + 2 * r + (e >> 1);
                            if (m < p.M) part[(team * p.M + m) * TN + n] = tot[f][r][e];
                        }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(seg_done);
        }
    } else {
        // ------------------------------------------------------------------ reducer
        int sg = 0;
        for (int tile = tile_first; tile <= tile_last; ++tile, ++sg) {
            const long long t_lo = (long long)tile * p.num_sb, t_hi = t_lo + p.num_sb;
            const int j_lo = (int)((t_lo > ub ? t_lo : ub) - ub), j_hi = (int)((t_hi < ue ? t_hi : ue) - ub);
            const int cnt = j_hi - j_lo;
            const bool whole = cnt == p.num_sb;
            // each lane owns CPL consecutive columns
            constexpr int CPL = TN / 32;
            const int n = CPL * lane, n_glob = tile * TN + n;
            const bool n_ok = n_glob < p.N;
            // the tile's contributors: the CTAs whose shares reach into [t_lo, t_hi) (every share has at least one unit)
            int c_first = cta, c_last = cta;
            while (c_first > 0 && shares.b[c_first] > t_lo) --c_first;
            while (c_last + 1 < P && shares.b[c_last + 1] < t_hi) ++c_last;
            // A tile shared between CTAs has one 64-bit word in the workspace: this launch's key in the upper 48 bits
            // and the number of contributors that have published their partial tile in the lower 16.  The key is
            // unique to the launch, so whatever an earlier use left there never counts.  The first contributor to
            // look at the word installs the key (compare-and-swap against what it saw; losing that race means somebody
            // else installed it); from then on the word only ever changes by atomic increments, and whoever finishes
            // the tile clears it, so a replay of the same launch (a captured graph) starts clean.
            unsigned long long *word = p.tags + tile;
            const int n_contrib = c_last - c_first + 1;
            const unsigned long long all_but_me = p.nonce | (unsigned long long)(n_contrib - 1);
            unsigned long long seen = 0ull;   // the word as this CTA last saw it
            // every lane reads the word itself (acquire), so its later reads of the partial tiles are ordered behind it
            auto others_published = [&]() {
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(word) : "memory");
                return seen == all_but_me;
            };
            // While the teams still work on this CTA's piece of a shared tile, see whether the other contributors
            // have published theirs already (the usual case for the piece a CTA works on last: its neighbour did
            // that tile first), and with one row fetch their partial tiles right away: the hand-over below
            // then needs no global round trip.
            bool early = false;
            constexpr int PRE_M = 1;
            float pre[PRE_M][2][CPL];   // [row][contributors before / after this CTA][column]
            auto fetch_others = [&]() {
                if (p.M <= PRE_M && c_last - cta <= 1) {
#pragma unroll
                    for (int m = 0; m < PRE_M; ++m) {
#pragma unroll
                        for (int c = 0; c < CPL; ++c) pre[m][0][c] = pre[m][1][c] = 0.f;
                        if (m < p.M && n_ok) {
                            for (int c = c_first; c <= c_last; ++c) {
                                if (c == cta) continue;
                                const float4 *src = reinterpret_cast<const float4 *>(p.slots + ((size_t)(tile + c) * p.M + m) * TN + n);
#pragma unroll
                                for (int q4 = 0; q4 < CPL / 4; ++q4) {
                                    const float4 a = __ldcg(src + q4);
                                    if (c > cta) {
                                        pre[m][1][4 * q4] += a.x; pre[m][1][4 * q4 + 1] += a.y; pre[m][1][4 * q4 + 2] += a.z; pre[m][1][4 * q4 + 3] += a.w;
                                    } else {
                                        pre[m][0][4 * q4] += a.x; pre[m][0][4 * q4 + 1] += a.y; pre[m][0][4 * q4 + 2] += a.z; pre[m][0][4 * q4 + 3] += a.w;
                                    }
                                }
                            }
                        }
                    }
                }
            };
            if (!whole) {
                if (sg == 0) pdl_wait_for_prerequisites();   // first touch of the workspace
                early = others_published();
                if ((seen & ~0xFFFFull) != p.nonce) {
                    if (lane == 0) {
                        unsigned long long old;
                        asm volatile("atom.relaxed.gpu.global.cas.b64 %0, [%1], %2, %3;" : "=l"(old) : "l"(word), "l"(seen), "l"(p.nonce) : "memory");
                    }
                    __syncwarp();
                    early = others_published();
                }
                if (early) fetch_others();
            }
            // Wait for the teams, and meanwhile keep an eye on the word: once every other contributor has published, their
            // partial tiles are fetched while the teams still work.
            {
                bool got = mbar_try_wait(seg_done, sg & 1);
                if (!got) {
                    const unsigned long long t0 = global_ns(), limit = p.wait_ns ? p.wait_ns : WAIT_LIMIT_NS;
                    const bool watch = !whole && !early;
                    while (true) {
                        // the look at the word is issued before the wait and consumed after it, so its L2 round trip
                        // runs beside the wait instead of delaying the moment the teams' arrival is noticed
                        unsigned long long peek = 0ull;
                        if (watch && !early) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(peek) : "l"(word));
                        if (mbar_try_wait_for(seg_done, sg & 1, 400u)) { got = true; break; }
                        if (watch && !early && peek == all_but_me && others_published()) { early = true; fetch_others(); }
                        if (*abort_flag) break;
                        if (global_ns() - t0 > limit) {
                            *abort_flag = 1;
                            atomicCAS(&g_tc_status, 0u, 0x330u);
                            break;
                        }
                    }
                }
                if (!got) break;
            }
            if (lane == 0 && tile == tile_last) MM_STAMP(5);
#ifdef WQ_MMA_PROFILE
            const unsigned long long prof_t0 = global_ns();
#endif
            if (whole && sg == 0) pdl_wait_for_prerequisites();   // first write to the output
            // this CTA's sum over its teams for row m of the tile
            auto own_row = [&](int m, float (&v)[CPL]) {
#pragma unroll
                for (int c = 0; c < CPL; ++c) v[c] = 0.f;
#pragma unroll
                for (int tm = 0; tm < MM_TEAMS; ++tm) {
                    if (cnt >= MM_TEAMS || (tm - j_lo % MM_TEAMS + MM_TEAMS) % MM_TEAMS < cnt) {
                        const float4 *src = reinterpret_cast<const float4 *>(part + (tm * p.M + m) * TN + n);
#pragma unroll
                        for (int c = 0; c < CPL / 4; ++c) {
                            const float4 a = src[c];
                            v[4 * c] += a.x; v[4 * c + 1] += a.y; v[4 * c + 2] += a.z; v[4 * c + 3] += a.w;
                        }
                    }
                }
            };
            auto write_row = [&](int m, const float (&v)[CPL]) {
                uint32_t o[CPL / 2];
                float fo[CPL];
#pragma unroll
                for (int c = 0; c < CPL / 2; ++c) {
                    float lo = v[2 * c], hi = v[2 * c + 1];
                    if (p.bias) {
                        lo += load_as_float(p.bias, BF16 ? ET_BF16 : ET_F16, n_glob + 2 * c);
                        hi += load_as_float(p.bias, BF16 ? ET_BF16 : ET_F16, n_glob + 2 * c + 1);
                    }
                    fo[2 * c] = lo; fo[2 * c + 1] = hi;
                    if constexpr (BF16) {
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi);
                        o[c] = *reinterpret_cast<uint32_t *>(&t2);
                    } else {
                        o[c] = pack_f16x2(lo, hi);
                    }
                }
                uint16_t *dst = static_cast<uint16_t *>(p.out) + (size_t)m * p.N + n_glob;
                if constexpr (Q8) *reinterpret_cast<uint2 *>(dst) = make_uint2(o[0], o[1]);
                else *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
                if (p.gather_n > 0) {
                    // the same row into every peer's window: packet i of a receive buffer = outputs 2 i, 2 i + 1 of the
                    // gathered [GPU][M][N] result.  A packet is one 8-byte store, so number and data arrive together and
                    // no fence is needed; the number tells the receiver that the packet belongs to this call.
                    const unsigned long long call = __ldcg(p.gather_calls) + 1ull;
                    const size_t elem = ((size_t)p.gather_rank * p.M + m) * p.N + n_glob;
                    const size_t off = (size_t)(call & 1ull) * p.gather_buf_bytes + (p.gather_f32 ? elem : elem >> 1) * 8;
                    for (int g = 0; g < p.gather_n; ++g) {
                        if (g == p.gather_rank && !p.gather_f32) continue;
                        uint2 *pk = reinterpret_cast<uint2 *>(p.gather_peer[g] + off);
                        if (p.gather_f32) {
#pragma unroll
                            for (int c = 0; c < CPL; ++c)
                                asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(pk + c), "r"(__float_as_uint(fo[c])), "r"((uint32_t)call) : "memory");
                        } else {
#pragma unroll
                            for (int c = 0; c < CPL / 2; ++c)
                                asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(pk + c), "r"(o[c]), "r"((uint32_t)call) : "memory");
                        }
                    }
                }
            };
            if (whole) {
                if (n_ok) {
                    for (int m = 0; m < p.M; ++m) {
                        float v[CPL];
                        own_row(m, v);
                        write_row(m, v);
                    }
                }
            } else {
                // A tile shared between CTAs.  A contributor that found all the OTHERS published when it looked (while its
                // teams were still working) adds its own part, still in shared memory, in contributor order and writes the
                // tile.  Otherwise it publishes its partial tile and counts itself in; whoever completes the count sums the
                // partial tiles and writes the tile.  No CTA ever waits for another.
                // sum in contributor order, this CTA's own part from shared memory
                auto finish = [&]() {
                    if (n_ok) {
                        for (int m = 0; m < p.M; ++m) {
                            float own[CPL], v[CPL];
                            own_row(m, own);
                            // four contributors' loads (the lane's eight columns each) are issued before the first is
                            // added, so their L2 round trips overlap; the sum stays in contributor order
#pragma unroll
                            for (int c = 0; c < CPL; ++c) v[c] = 0.f;
                            for (int c0 = c_first; c0 <= c_last; c0 += 4) {
                                float4 a[4][CPL / 4];
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    const int c = c0 + u;
#pragma unroll
                                    for (int q4 = 0; q4 < CPL / 4; ++q4) a[u][q4] = make_float4(own[4 * q4], own[4 * q4 + 1], own[4 * q4 + 2], own[4 * q4 + 3]);
                                    if (c <= c_last && c != cta) {   // written by other SMs: read at L2
                                        const float4 *src = reinterpret_cast<const float4 *>(p.slots + ((size_t)(tile + c) * p.M + m) * TN + n);
#pragma unroll
                                        for (int q4 = 0; q4 < CPL / 4; ++q4) a[u][q4] = __ldcg(src + q4);
                                    }
                                }
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    if (c0 + u > c_last) break;
#pragma unroll
                                    for (int q4 = 0; q4 < CPL / 4; ++q4) {
                                        v[4 * q4] += a[u][q4].x; v[4 * q4 + 1] += a[u][q4].y; v[4 * q4 + 2] += a[u][q4].z; v[4 * q4 + 3] += a[u][q4].w;
                                    }
                                }
                            }
                            write_row(m, v);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) *word = 0ull;
                };
                if (early && p.M <= PRE_M && c_last - cta <= 1) {
                    // the others' sums are in registers: (before + own) + after is finish()'s order exactly when at
                    // most one contributor comes after this CTA, so the bits do not depend on who finishes the tile
                    if (n_ok) {
#pragma unroll
                        for (int m = 0; m < PRE_M; ++m) {
                            if (m >= p.M) break;
                            float own[CPL], v[CPL];
                            own_row(m, own);
#pragma unroll
                            for (int c = 0; c < CPL; ++c) v[c] = (pre[m][0][c] + own[c]) + pre[m][1][c];
                            write_row(m, v);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) *word = 0ull;
                } else if (early) {
                    finish();
                } else {
                    if (n_ok) {
                        for (int m = 0; m < p.M; ++m) {
                            float v[CPL];
                            own_row(m, v);
                            float4 *dst = reinterpret_cast<float4 *>(p.slots + ((size_t)(tile + cta) * p.M + m) * TN + n);
#pragma unroll
                            for (int c = 0; c < CPL / 4; ++c) dst[c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                        }
                    }
                    // Publish: the warp barrier orders every lane's stores before lane 0's increment, whose release half
                    // makes them visible with the new count (release is cumulative) and whose acquire half orders the
                    // reads of finish() behind every earlier contributor's increment (they form one chain of
                    // read-modify-writes on the word).  The contributor that brings the count to n_contrib finishes the
                    // tile: exactly one does, and it waits for nobody.
                    __syncwarp();
                    unsigned long long now = 0ull;
                    if (lane == 0) {
                        asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], %2;" : "=l"(now) : "l"(word), "l"(1ull) : "memory");
                        now += 1ull;
                    }
                    now = __shfl_sync(0xffffffffu, now, 0);
                    __syncwarp();
                    if (now == (p.nonce | (unsigned long long)n_contrib)) finish();
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(seg_free);
#ifdef WQ_MMA_PROFILE
            if (lane == 0 && !whole) g_mm_prof[7][cta < 160 ? cta : 159] += global_ns() - prof_t0;
#endif
        }
        if (lane == 0) MM_STAMP(6);
    }
}

// ---- the tile-packed weight layout --------------------------------------------------------------
// int4 weights [K,N] re-laid as blocks of 16 KB, one per (tile of 256 columns, stage of 128 K rows),
// tile-major ([tile][stage]) so that a CTA's stream-K share is one contiguous range.  Inside a block
// the order is [warp quarter wq = 64 columns][step st = 16 K rows][lane = (g, t)][word r]: the 16 bytes
// a lane of the decode kernel needs for one step, so a step is one 16-byte shared-memory load and no
// byte shuffling.  Word r covers the lane's columns c + 2r, c + 2r + 1 (c = 256 tile + 64 wq + 8 g) and
// rows k + 2t, k + 2t + 1, k + 2t + 8, k + 2t + 9 (k = 128 stage + 16 st): nibble 0 / 4 = column 2r at
// rows 2t / 2t+1, nibble 1 / 5 = column 2r+1, nibbles 2 / 6 and 3 / 7 the same at rows 2t+8 / 2t+9.
// Columns beyond N and rows beyond K are zero.
__host__ __device__ inline void nz_source(int nib, int &dk, int &dc) {
    dc = nib & 1;                                  // column 2r + dc
    dk = ((nib >> 2) & 1) + ((nib >> 1) & 1) * 8;  // row 2t + dk
}

__global__ void wq_pack_nz_kernel(const uint8_t *w, uint32_t *out, int K, int N, int num_sb, long long words) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    const int r = (int)(i & 3), lane = (int)((i >> 2) & 31), st = (int)((i >> 7) & 7), wq = (int)((i >> 10) & 3);
    const long long blk = i >> 12;
    const int sb = (int)(blk % num_sb), tile = (int)(blk / num_sb);
    const int g = lane >> 2, t = lane & 3;
    const int c = tile * 256 + wq * 64 + 8 * g + 2 * r, k = sb * 128 + st * 16 + 2 * t;
    uint32_t word = 0;
#pragma unroll
    for (int nib = 0; nib < 8; ++nib) {
        int dk, dc;
        nz_source(nib, dk, dc);
        const int kk = k + dk, cc = c + dc;
        if (kk < K && cc < N) {
            const size_t idx = (size_t)kk * N + cc;
            word |= (uint32_t)((w[idx >> 1] >> ((idx & 1) * 4)) & 0xF) << (4 * nib);
        }
    }
    out[i] = word;
}

// Back to the caller's layout (one thread per 8 consecutive columns of a row = one packed word).
__global__ void wq_unpack_nz_kernel(const uint32_t *nz, uint32_t *out, int K, int N, int num_sb) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int wpr = N / 8;
    if (i >= (long long)K * wpr) return;
    const int k = (int)(i / wpr), c = (int)(i % wpr) * 8;
    const int tile = c >> 8, wq = (c >> 6) & 3, g = (c >> 3) & 7;
    const int sb = k >> 7, st = (k >> 4) & 7, kr = k & 15, t = (kr & 7) >> 1;
    const int nib_base = (kr & 1) * 4 + (kr >> 3) * 2;   // + dc
    const uint4 v = *reinterpret_cast<const uint4 *>(nz + ((((size_t)tile * num_sb + sb) * 4 + wq) * 8 + st) * 128 + (4 * g + t) * 4);
    const uint32_t src[4] = {v.x, v.y, v.z, v.w};
    uint32_t word = 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        word |= ((src[r] >> (4 * nib_base)) & 0xFu) << (8 * r);
        word |= ((src[r] >> (4 * (nib_base + 1))) & 0xFu) << (8 * r + 4);
    }
    out[i] = word;
}

int mm_sm_count() {
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] { for (int &c : cached) c = 0; });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    dev &= 63;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        cached[dev] = n;
    }
    return cached[dev];
}

struct MmPlan {
    int mf, tiles, num_sb, gsb, P;
    bool xpre;               // activations converted once per call by wq_mma_activation_kernel
    long long total_u;
    uint64_t slot_bytes, tag_bytes, xf_bytes;
    MmShares shares;
};

// Shares of the (tile, stage) space: equal by default.  When there are more CTAs than tiles and a share is shorter than
// a tile, some CTAs lie wholly inside one tile ("interior"), and such a tile then has two contributors that finish at
// the very end of the kernel -- the interior one and the one whose share ends in the tile -- so neither finds the
// other's partial tile published and both go through the slower hand-over.  B200_QMM_WQ_STAGGER=<stages> makes the
// interior shares that much shorter (the others correspondingly longer), so that the interior CTA publishes before the
// other one finishes.  Measured on the 8192 x 28672 call it does not pay: 26.0 us with equal shares, 26.1-26.4 with
// 4.5 stages, 26.5-26.6 with 6 (the longer shares cost what the quicker hand-over gains), so the default is 0.
void mm_fill_shares(MmPlan &pl) {
    const long long U = pl.total_u;
    const int P = pl.P, S = pl.num_sb;
    for (int c = 0; c <= P; ++c) pl.shares.b[c] = (long long)c * U / P;
    double stagger = 0.0;
    if (const char *e = getenv("B200_QMM_WQ_STAGGER")) stagger = atof(e);
    const double even = (double)U / P;
    if (stagger <= 0.0 || P <= pl.tiles || even >= S || even < 4.0 * stagger) return;
    auto walk = [&](double ls, long long *b) {
        double pos = 0.0;
        int c = 0;
        while (pos < (double)U - 1e-6 && c < MM_MAX_CTAS) {
            const double rest = S - fmod(pos, (double)S);            // stages left in the current tile
            if (b) b[c] = llround(pos);
            pos += rest > ls + 1e-9 ? ls - stagger : ls;             // cannot reach the tile's end: interior, shorter
            ++c;
        }
        return c;
    };
    // the shortest long share with which P CTAs cover everything
    double lo = even, hi = even + stagger;
    if (walk(hi, nullptr) > P) return;
    for (int it = 0; it < 60; ++it) {
        const double mid = 0.5 * (lo + hi);
        if (walk(mid, nullptr) > P) lo = mid; else hi = mid;
    }
    long long b[MM_MAX_CTAS + 1];
    const int used = walk(hi, b);
    if (used != P) return;      // fewer CTAs would do: keep the equal shares
    b[P] = U;
    for (int c = 0; c < P; ++c)
        if (b[c + 1] <= b[c]) return;   // every share needs at least one unit
    for (int c = 0; c <= P; ++c) pl.shares.b[c] = b[c];
}

MmPlan mm_make_plan(const MatmulArgs &p) {
    MmPlan pl{};
    pl.mf = p.M <= 8 ? 1 : 2;
    const int tile_n = p.b_type == ET_I8 ? 128 : 256;
    pl.tiles = (int)((p.N + tile_n - 1) / tile_n);
    pl.num_sb = (int)((p.K + MM_SBK - 1) / MM_SBK);
    pl.gsb = p.group < p.K ? (int)(p.group / MM_SBK) : pl.num_sb;
    pl.total_u = (long long)pl.tiles * pl.num_sb;
    const int sms = mm_sm_count();
    pl.P = (int)(pl.total_u < sms ? pl.total_u : sms);
    // Small problems: with one whole tile per CTA every tile is finished where it was computed and the
    // finalize kernel (about 3 us at this scale) is not launched.  Worth it when streaming a whole tile
    // into one SM (about 50 GB/s) costs less than an even share plus that launch.
    // B200_QMM_WQ_WHOLE_TILES=0|1 overrides.
    if (pl.tiles <= sms && pl.tiles < pl.P) {
        const double tile_bytes = (double)p.K * tile_n * (p.b_type == ET_I8 ? 1.0 : 0.5);
        bool whole = tile_bytes / 50e9 < tile_bytes * pl.tiles / pl.P / 50e9 + 3e-6;
        if (const char *e = getenv("B200_QMM_WQ_WHOLE_TILES")) whole = atoi(e) != 0;
        if (whole) pl.P = pl.tiles;
    }
    // Shares that do not straddle tiles: with a few CTAs fewer, every share can be an equal divisor (or
    // multiple) of a tile's stages, so each CTA adds to one tile only and fewer partial tiles are written and
    // summed (4096 x 4096 int4 at M = 16: 16.7 us on 148 CTAs, 14.9 us on 128).  Take the largest such CTA
    // count within 15 % of the SM count.  B200_QMM_WQ_MMA_P=<n> overrides.
    if (pl.P == sms && pl.total_u < 8LL * sms) {   // small problems only: large ones are bound by the work per SM
        for (int c = sms; c >= sms - sms * 15 / 100; --c) {
            if (pl.total_u % c != 0) continue;
            const long long share = pl.total_u / c;
            if (pl.num_sb % share == 0 || share % pl.num_sb == 0) { pl.P = c; break; }
        }
    }
    if (const char *e = getenv("B200_QMM_WQ_MMA_P")) { const int v = atoi(e); if (v >= 1 && v <= sms && v <= pl.total_u) pl.P = v; }
    if (pl.P > MM_MAX_CTAS) pl.P = MM_MAX_CTAS;
    mm_fill_shares(pl);
    pl.slot_bytes = align_up_u64((uint64_t)(pl.tiles + pl.P) * p.M * tile_n * sizeof(float), 256);
    pl.tag_bytes = align_up_u64((uint64_t)pl.tiles * sizeof(unsigned long long), 256);
    // rows from which the activations are converted by the pre-pass instead of inside the kernel (B200_QMM_WQ_XPRE_M)
    int xpre_m = 5;
    if (const char *e = getenv("B200_QMM_WQ_XPRE_M")) xpre_m = atoi(e) > 0 ? atoi(e) : 1;
    pl.xpre = pl.mf == 2 || p.M >= xpre_m;
    pl.xf_bytes = pl.xpre ? align_up_u64((uint64_t)pl.num_sb * (pl.mf * 2048 + 128), 256) : 0;
    return pl;
}

constexpr int MM_SMEM_LIMIT = 232448;

// A 64-bit value no earlier launch of this process has used and that stale workspace contents match with
// probability 2^-64: a counter run through a bijective mixer, seeded once from the clock and an address.
unsigned long long mm_next_nonce() {
    static std::atomic<unsigned long long> counter{[] {
        unsigned long long seed = (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count();
        int probe = 0;
        return seed ^ ((unsigned long long)(uintptr_t)&probe << 17) ^ 0x9E3779B97F4A7C15ull;
    }()};
    unsigned long long z = counter.fetch_add(0x9E3779B97F4A7C15ull) + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z ? z : 1ull;
}

// Ring depth: every slot must belong to one team, so the depth is c x teams.  Three slots per team hide
// the HBM round trip (one being read, the others in flight); take the deepest ring up to that which fits
// beside the partial tiles.
template <int MF>
int mm_ring_slots(int M) {
    for (int c = 3; c >= 2; --c)
        if (MmSmem<MF>::total(c * MM_TEAMS, M) <= MM_SMEM_LIMIT) return c * MM_TEAMS;
    return 0;
}

template <bool Q8, bool BF16, int MF, bool NZ>
cudaError_t mm_launch_one(const CUtensorMap &tw, MmParams mp, const MmShares &shares, int P, cudaStream_t s) {
    using L = MmSmem<MF>;
    static_assert(L::SLOT % 1024 == 0, "slots keep the swizzle alignment");
    mp.ns = mm_ring_slots<MF>(mp.M);
    if (mp.ns == 0) return cudaErrorInvalidValue;
    const int smem = L::total(mp.ns, mp.M);
    auto kern = wq_mma_kernel<Q8, BF16, MF, NZ>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    // Programmatic stream serialisation (see pdl_wait_for_prerequisites).  B200_QMM_PDL=0 launches the plain way;
    // B200_QMM_PDL=2 additionally lets the weight stream start before the preceding kernel has completed, which is
    // only right when that kernel does not write this call's weights, scales or offsets.
    static const int pdl = [] { const char *e = getenv("B200_QMM_PDL"); return e ? atoi(e) : 1; }();
    mp.weights_early = pdl >= 2 ? 1 : 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)P);
    cfg.blockDim = dim3(MM_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl >= 1 ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, mp, shares);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

#ifdef WQ_MMA_PROFILE
// Copies the stamps of the launches so far to `host` (8 x 160 values) and clears rows 4 and 7.
extern "C" __attribute__((visibility("default"))) int aclnnB200DecodeProfile(unsigned long long *host) {
    if (cudaMemcpyFromSymbol(host, g_mm_prof, sizeof(g_mm_prof)) != cudaSuccess) return 1;
    static unsigned long long zero[8][160] = {};
    return cudaMemcpyToSymbol(g_mm_prof, zero, sizeof(zero)) == cudaSuccess ? 0 : 1;
}
#endif

namespace {
thread_local DecodeGather tl_gather{};
thread_local bool tl_gather_set = false, tl_gather_consumed = false;
}  // namespace
void wq_mma_set_gather(const DecodeGather *g) {
    tl_gather_set = g != nullptr && g->nranks >= 2 && g->nranks <= MM_MAX_PEERS && g->rank < g->nranks;
    if (tl_gather_set) tl_gather = *g;
    tl_gather_consumed = false;
}
bool wq_mma_gather_consumed() { return tl_gather_consumed; }

bool wq_mma_supported(const MatmulArgs &p) {
    if (p.epilogue != EPI_PLAIN || !p.scale || p.a_scale || p.b_scale) return false;
    if (p.batch != 1 || p.b_transposed || p.accumulate || p.M < 1 || p.M > MM_MAX_ROWS) return false;
    if (p.a_type != ET_F16 && p.a_type != ET_BF16) return false;
    if (p.b_type != ET_I4 && p.b_type != ET_I8) return false;
    if (p.b_nz && p.b_type != ET_I4) return false;
    if (p.sc_type != p.a_type || p.out_type != p.a_type || (p.bias && p.bias_type != p.a_type)) return false;
    if (p.K % 8 != 0 || p.K < MM_SBK || p.N % (p.b_type == ET_I4 ? 32 : 16) != 0) return false;
    if (p.group < p.K && (p.group % MM_SBK != 0 || p.K % p.group != 0)) return false;
    if (p.N > (1 << 24) || p.K > (1 << 24)) return false;
    if (const char *e = getenv("B200_QMM_WQ_MMA")) {
        if (atoi(e) == 0) return false;
    }
    return true;
}

// Some row counts on weights in the caller's layout go to the kernel that takes the activations as they are
// (wq_rows.cu), where it measured faster on 8192 x 28672 (us per call, this kernel / that one): 3 rows 29.8 / 32.7,
// 4 rows 31.5 / 33.0, 5 rows 33.8 / 33.5, 6 rows 35.3 / 34.3, 8 rows 37.8 / 35.5, 9 rows 43.6 / 46.3, 12 rows 47.8 / 48.7,
// 16 rows 53.0 / 50.5.  B200_QMM_WQ_ROWS=0 keeps everything here, =<m> sends m rows and more there.
inline bool mm_use_rows_kernel(const MatmulArgs &p) {
    if (p.b_nz || tl_gather_set || !wq_rows_supported(p)) return false;   // the gathering epilogue lives in this kernel
    if (const char *e = getenv("B200_QMM_WQ_ROWS")) return atoi(e) > 0 && p.M >= atoi(e);
    return (p.M >= 5 && p.M <= 8) || p.M >= 13;
}

uint64_t wq_mma_workspace_bytes(const MatmulArgs &p) {
    if (mm_use_rows_kernel(p)) return wq_rows_workspace_bytes(p);
    const MmPlan pl = mm_make_plan(p);
    return pl.slot_bytes + pl.tag_bytes + pl.xf_bytes;
}

cudaError_t launch_wq_mma(const MatmulArgs &p, cudaStream_t s) {
    if (mm_use_rows_kernel(p)) return launch_wq_rows(p, s);
    const MmPlan pl = mm_make_plan(p);
    if (p.workspace_bytes < pl.slot_bytes + pl.tag_bytes + pl.xf_bytes || !p.workspace) return cudaErrorInvalidValue;
    // TMA / bulk-copy sources, the 16-byte activation, scale and offset loads, the 16-byte output stores and
    // the float4 partial tiles all need 16-byte aligned bases (every row pitch already is a multiple of 16 bytes).
    if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15) ||
        (reinterpret_cast<uintptr_t>(p.scale) & 15) || (reinterpret_cast<uintptr_t>(p.offset) & 15) ||
        (reinterpret_cast<uintptr_t>(p.out) & 15) || (reinterpret_cast<uintptr_t>(p.workspace) & 15))
        return cudaErrorMisalignedAddress;
    const bool bf = p.a_type == ET_BF16, q8 = p.b_type == ET_I8;
    CUtensorMap tw{};
    if (!p.b_nz) {
        // No L2 promotion: every byte of the weight stream is used exactly once by exactly one CTA, and
        // fetching wider L2 lines than asked for measurably slows the stream down.
        const uint64_t row_bytes = q8 ? (uint64_t)p.N : (uint64_t)p.N / 2;
        if (!make_map(&tw, p.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, row_bytes, p.K, row_bytes, 128, MM_SBK, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_NONE))
            return cudaErrorInvalidValue;
    }

    MmParams mp{};
    mp.out = p.out;
    mp.slots = (float *)p.workspace;
    mp.tags = (unsigned long long *)((char *)p.workspace + pl.slot_bytes);
    mp.nonce = mm_next_nonce() & ~0xFFFFull;
    if (mp.nonce == 0ull) mp.nonce = 1ull << 16;
    if (pl.xpre) {
        uint8_t *xf = (uint8_t *)p.workspace + pl.slot_bytes + pl.tag_bytes;
        const uint16_t *xa = (const uint16_t *)p.a;
        if (pl.mf == 2) {
            if (p.a_type == ET_BF16) wq_mma_activation_kernel<true, 2><<<pl.num_sb, 32, 0, s>>>(xa, xf, (int)p.M, (int)p.K);
            else wq_mma_activation_kernel<false, 2><<<pl.num_sb, 32, 0, s>>>(xa, xf, (int)p.M, (int)p.K);
        } else {
            if (p.a_type == ET_BF16) wq_mma_activation_kernel<true, 1><<<pl.num_sb, 32, 0, s>>>(xa, xf, (int)p.M, (int)p.K);
            else wq_mma_activation_kernel<false, 1><<<pl.num_sb, 32, 0, s>>>(xa, xf, (int)p.M, (int)p.K);
        }
        count_launch();
        mp.xf = xf;
    }
    mp.x = p.a;
    mp.scale = p.scale; mp.offset = p.offset; mp.bias = p.bias;
    mp.wnz = p.b_nz ? (const uint8_t *)p.b : nullptr;
    mp.x_bf16 = bf ? 1 : 0;
    mp.M = (int)p.M; mp.N = (int)p.N; mp.K = (int)p.K;
    mp.num_sb = pl.num_sb; mp.total_u = pl.total_u; mp.gsb = pl.gsb;
    mp.tile_n = q8 ? 128 : 256;
    // gathering epilogue asked for by the calling thread (wq_mma_set_gather), if the receive buffers hold the result
    if (tl_gather_set && (uint64_t)tl_gather.nranks * p.M * p.N * (tl_gather.f32 ? 8 : 4) <= tl_gather.buf_bytes && (p.N & 1) == 0 &&
        !(tl_gather.f32 && p.bias)) {   // partial results must not each carry the bias
        mp.gather_n = (int)tl_gather.nranks; mp.gather_rank = (int)tl_gather.rank;
        for (int g = 0; g < mp.gather_n; ++g) mp.gather_peer[g] = (unsigned long long)(uintptr_t)tl_gather.peer[g];
        mp.gather_buf_bytes = tl_gather.buf_bytes;
        mp.gather_f32 = tl_gather.f32 ? 1 : 0;
        mp.gather_calls = tl_gather.calls;
        tl_gather_consumed = true;
    }
    // test hooks: B200_QMM_TEST_WAIT_LIMIT_NS=<n> gives every wait of the decode kernel n nanoseconds instead of about a
    // second; B200_QMM_TEST_DROP_STAGE=1 makes CTA 0 leave out the copy of its first stage, so that the consumers' wait
    // for it is a wait for something that never comes
    if (const char *e = getenv("B200_QMM_TEST_WAIT_LIMIT_NS")) mp.wait_ns = strtoull(e, nullptr, 10);
    if (const char *e = getenv("B200_QMM_TEST_DROP_STAGE")) mp.test_drop = atoi(e);

    cudaError_t e;
#define MM_GO(Q8_, NZ_) (pl.mf == 1 ? (bf ? mm_launch_one<Q8_, true, 1, NZ_>(tw, mp, pl.shares, pl.P, s) : mm_launch_one<Q8_, false, 1, NZ_>(tw, mp, pl.shares, pl.P, s)) \
                                    : (bf ? mm_launch_one<Q8_, true, 2, NZ_>(tw, mp, pl.shares, pl.P, s) : mm_launch_one<Q8_, false, 2, NZ_>(tw, mp, pl.shares, pl.P, s)))
    if (q8) e = MM_GO(true, false);
    else if (p.b_nz) e = MM_GO(false, true);
    else e = MM_GO(false, false);
#undef MM_GO
    return e;
}

// ---- the tile-packed layout: size, pack, unpack -----------------------------------------------------
uint64_t wq_nz_bytes(int64_t K, int64_t N) {
    const uint64_t tiles = (uint64_t)(N + MM_TILE_N - 1) / MM_TILE_N, num_sb = (uint64_t)(K + MM_SBK - 1) / MM_SBK;
    return tiles * num_sb * MM_W_BYTES;
}

cudaError_t launch_wq_pack_nz(const void *w_nd, void *w_nz, int64_t K, int64_t N, cudaStream_t s) {
    if ((N & 1) || K < 1 || N < 1 || K > (1 << 24) || N > (1 << 24)) return cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(w_nz) & 15) return cudaErrorMisalignedAddress;
    const long long words = (long long)(wq_nz_bytes(K, N) / 4);
    const int num_sb = (int)((K + MM_SBK - 1) / MM_SBK);
    wq_pack_nz_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>((const uint8_t *)w_nd, (uint32_t *)w_nz, (int)K, (int)N, num_sb, words);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_wq_unpack_nz(const void *w_nz, void *w_nd, int64_t K, int64_t N, cudaStream_t s) {
    if ((N & 7) || K < 1 || N < 1) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(w_nz) & 15) || (reinterpret_cast<uintptr_t>(w_nd) & 3)) return cudaErrorMisalignedAddress;
    const long long words = (long long)K * (N / 8);
    const int num_sb = (int)((K + MM_SBK - 1) / MM_SBK);
    wq_unpack_nz_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>((const uint32_t *)w_nz, (uint32_t *)w_nd, (int)K, (int)N, num_sb);
    count_launch();
    return cudaGetLastError();
}

void wq_mma_device_status_reset() {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(z));
}

unsigned int wq_mma_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    return v;
}

}  // namespace qmm
