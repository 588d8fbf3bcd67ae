// Native block-scaled MX matmul (sm_100a): tcgen05.mma.kind::mxf8f6f4.block_scale with the e8m0 scales
// in tensor memory, fp32 accumulators in tensor memory, operands straight from TMA-swizzled shared memory.
//
//   out[M,N] = sum_k  A[m,k] * 2^(sA[m,k/32]-127) * B[k,n] * 2^(sB[k/32,n]-127)
//
// Operands as the tensor core wants them:
//   * A [M,K], K contiguous: the K-major operand form, one TMA box of 128 rows x 128 bytes per stage.
//   * B [K,N], N contiguous: the MN-major operand form, which the instruction takes for 8-bit element
//     types only.  fp8 B goes in as it is.  fp4 elements (two per byte) are first widened to the fp8 e4m3
//     byte of the same value (every e2m1 value is exact in e4m3) by one streaming pass into the workspace;
//     after that both kinds are the same [K,N] byte matrix and no transpose is needed anywhere.  (The
//     reference transposes B and re-lays both scale tensors on every call, cuda/src/ops/matmul.cu:560-577.)
//     fp4 A is widened the same way.
//   * Scales: the instruction reads one e8m0 byte per (row, 32-element K block) from tensor memory,
//     where a 128-row x 4-block group is laid out as 32 lanes x 16 bytes: byte (r % 32) * 16 + (r / 32) * 4
//     + block.  That is the layout the reference computes in k_swizzle_scale (matmul.cu:75-84).  A small
//     pass re-lays sA [M,K/32] and sB [K/32,N] into such 512-byte groups in the workspace; the main
//     kernel brings one group of A and two of B per stage into shared memory with plain bulk copies and
//     moves them to tensor memory with tcgen05.cp, in order ahead of the stage's four MMAs.
//
// Kernel: persistent, one CTA per SM, 320 threads.  Warp 0 = TMA producer (ring of 4 stages of 128 K),
// warp 1 = MMA issuer and tensor-memory owner, warps 2-9 = epilogue (two sets of four warps, 128 columns
// each).  Tile = 128 rows x 256 columns with one accumulator of 256 tensor-memory columns; the scale groups take
// 2 x 16 further columns.  (The tile width is a launch parameter: up to 240 columns two accumulators fit and the
// epilogue of one tile overlaps the MMAs of the next; the weight boxes and scale groups stay 256 columns wide, the
// columns beyond the tile belong to the next one and are not multiplied.  mx_layout says why 256 is the default.)
// Every wait is bounded and records a code in the device status word.
//
// Replaces aclnnMatmulMxFp8Hw / aclnnMatmulMxFp4Hw of the reference (cuBLASLt VEC32_UE8M0 behind per-call
// transpose and scale passes, cuda/src/ops/matmul.cu:538-597,657-730).
#include <cstdlib>

#include "tc_common.cuh"

namespace qmm {
namespace {

constexpr int MX_M = 128, MX_N = 256, MX_BK = 128;

// MH = row halves of a tile: 1 = 128 rows (ring of 4 stages), 2 = 256 rows as two accumulators over one weight tile
// (ring of 3 stages): the weight tile is then fetched once for twice the rows, which is what the kernel is short of.
template <int MH>
struct MxSmem {
    static constexpr int STAGES = MH == 1 ? 4 : 3;
    static constexpr int X_BYTES = MH * MX_M * MX_BK;       // 16 KB per 128 rows x 128 K bytes, 128-byte swizzle
    static constexpr int W_BYTES = MX_N * MX_BK;            // 32 KB: two boxes of 128 columns x 128 K rows
    static constexpr int SFA_OFF = X_BYTES + W_BYTES;       // 512 B per 128 rows: their scales for 4 K blocks
    static constexpr int SFB_OFF = SFA_OFF + MH * 512;      // 1024 B: scales of 256 columns x 4 K blocks
    static constexpr int STAGE_BYTES = (SFB_OFF + 1024 + 1023) / 1024 * 1024;
    static constexpr int PAYLOAD = X_BYTES + W_BYTES + MH * 512 + 1024;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 4;
    static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
    static constexpr int TOTAL = MISC_OFF + 16 + 1024;
};
static_assert(MxSmem<1>::TOTAL <= 232448 && MxSmem<2>::TOTAL <= 232448, "shared memory budget of one CTA");

struct MxParams {
    void *out;
    int out_type;
    int M, N, K;
    int m_tiles, tiles, num_kb;     // tiles are numbered n_tile * m_tiles + m_tile; num_kb = K / 128
    int tile_n;                     // output columns per tile: 256, or less (a multiple of 16)
    int nacc;                       // accumulators in tensor memory, tile_n columns apart
    const uint8_t *sfa;             // [128-row group][k chunk][512] scale groups of A
    const uint8_t *sfb;             // [k chunk][n_tile][2][512] scale groups of B: columns tile_n * n_tile + 128 * h ...
    int n128e;                      // 2 * n_tiles
};

constexpr uint32_t MX_TMEM_COLS = 512;
constexpr uint32_t MX_SF_COL = 480;   // scale groups live behind the accumulators: two buffers of 16 columns

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 tensor-memory columns of lanes 0-31, repeated in all four lane quarters.
__device__ __forceinline__ void sf_copy(uint32_t taddr, uint32_t smem_addr) {
    // no swizzle, rows 16 bytes apart, 8-row groups 128 bytes apart, descriptor version 1
    const uint64_t desc = (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(16u >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mx_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                       uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate) : "memory");
}
// Block-scaled instruction descriptor: A/B formats (0 = e4m3, 1 = e5m2), A K-major, B MN-major, e8m0 scales,
// N >> 3 at bit 17, M >> 4 at bit 24; the scale byte of the K block (0-3) of both operands at bits 4 and 29.
__host__ __device__ constexpr uint32_t mx_idesc(int a_fmt, int b_fmt, int m, int n) {
    return ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(n >> 3) << 17) | (1u << 23) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void mx_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

template <int MH>
__global__ void __launch_bounds__(320, 1)
mx_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const MxParams p, const uint32_t idesc) {
    using L = MxSmem<MH>;
    constexpr int MX_STAGES = L::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    auto a_tile = [&](int s) { return base + s * L::STAGE_BYTES; };
    auto b_tile = [&](int s) { return base + s * L::STAGE_BYTES + L::X_BYTES; };
    auto bar_full = [&](int s) { return base + L::BAR_OFF + 8 * s; };
    auto bar_empty = [&](int s) { return base + L::BAR_OFF + 8 * (MX_STAGES + s); };
    auto bar_acc_full = [&](int a) { return base + L::BAR_OFF + 8 * (2 * MX_STAGES + a); };
    auto bar_acc_empty = [&](int a) { return base + L::BAR_OFF + 8 * (2 * MX_STAGES + 2 + a); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen_base + L::MISC_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + L::MISC_OFF + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MX_STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(bar_acc_full(a), 1); mbar_init(bar_acc_empty(a), 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void *)tmem_slot), MX_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto tile_geom = [&](int tile, int &n0, int &m0) {
        n0 = (tile / p.m_tiles) * p.tile_n;
        m0 = (tile % p.m_tiles) * (MH * MX_M);
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
                int n0, m0;
                tile_geom(tile, n0, m0);
                const uint8_t *sfa = p.sfa + (size_t)(m0 / MX_M) * p.num_kb * 512;   // the tile's first 128-row group
                const uint8_t *sfb = p.sfb + (size_t)(tile / p.m_tiles) * 1024;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % MX_STAGES;
                    if (it >= MX_STAGES && !mbar_wait(bar_empty(s), ((it / MX_STAGES) - 1) & 1, abort_flag, 0x401u)) { ok = false; break; }
                    mbar_expect_tx(bar_full(s), L::PAYLOAD);
                    const int k = kb * MX_BK;
#pragma unroll
                    for (int h = 0; h < MH; ++h) {
                        tma_load_2d(a_tile(s) + h * 16384, &tm_a, bar_full(s), k, m0 + h * MX_M);
                        bulk_g2s(a_tile(s) + L::SFA_OFF + h * 512, sfa + ((size_t)h * p.num_kb + kb) * 512, 512, bar_full(s));
                    }
                    tma_load_2d(b_tile(s), &tm_b, bar_full(s), n0, k);
                    tma_load_2d(b_tile(s) + 16384, &tm_b, bar_full(s), n0 + 128, k);
                    bulk_g2s(a_tile(s) + L::SFB_OFF, sfb + (size_t)kb * p.n128e * 512, 1024, bar_full(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, ti = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++ti) {
                const int ab = ti % p.nacc;
                const uint32_t d_tmem = tmem_base + (uint32_t)(ab * p.tile_n);
                if (ti >= p.nacc) {   // the epilogue has drained this accumulator's previous tile
                    if (!mbar_wait(bar_acc_empty(ab), (ti / p.nacc - 1) & 1, abort_flag, 0x402u)) { ok = false; break; }
                    tc_fence_after();
                }
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % MX_STAGES;
                    if (!mbar_wait(bar_full(s), (it / MX_STAGES) & 1, abort_flag, 0x403u)) { ok = false; break; }
                    tc_fence_after();
                    // this stage's scale groups: A (128 rows) -> 4 columns (the second row half: the last 4 of the 16),
                    // B (256 columns) -> 8 columns
                    const uint32_t sf = tmem_base + MX_SF_COL + (uint32_t)(it & 1) * 16u;
                    sf_copy(sf, a_tile(s) + L::SFA_OFF);
                    if constexpr (MH == 2) sf_copy(sf + 12, a_tile(s) + L::SFA_OFF + 512);
                    sf_copy(sf + 4, a_tile(s) + L::SFB_OFF);
                    sf_copy(sf + 8, a_tile(s) + L::SFB_OFF + 512);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t b_desc = smem_desc(b_tile(s) + kk * 4096, 16384, 1024);
#pragma unroll
                        for (int h = 0; h < MH; ++h) {     // both row halves multiply the same weight tile
                            const uint64_t a_desc = smem_desc(a_tile(s) + h * 16384 + kk * 32, 16, 1024);
                            mx_mma(d_tmem + (uint32_t)(h * p.tile_n), a_desc, b_desc, idesc | ((uint32_t)kk << 4) | ((uint32_t)kk << 29),
                                   sf + (h ? 12u : 0u), sf + 4, (kb > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    tc_commit(bar_empty(s));
                }
                if (ok) tc_commit(bar_acc_full(ab));
            }
        }
    } else {
        // epilogue: a warp's tensor-memory lane quarter = 32 rows.  One row half: the two sets of four warps take half of
        // the columns each; two row halves: a set takes a row half (its accumulator) with all the columns
        const int eset = (warp - 2) >> 2, q = warp & 3;
        const int half = MH == 1 ? p.tile_n >> 1 : p.tile_n;   // columns per epilogue set (a multiple of 8)
        const int row = (MH == 2 ? eset * MX_M : 0) + q * 32 + lane, cb = MH == 1 ? eset * half : 0;
        const uint32_t acc_off = MH == 2 ? (uint32_t)(eset * p.tile_n) : 0u;
        int ti = 0;
        for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++ti) {
            int n0, m0;
            tile_geom(tile, n0, m0);
            const int m = m0 + row;
            const bool m_ok = m < p.M;
            const int ab = ti % p.nacc;
            if (!mbar_wait(bar_acc_full(ab), (ti / p.nacc) & 1, abort_flag, 0x405u)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * p.tile_n) + acc_off + cb;
            const int esz = p.out_type == ET_F32 ? 4 : 2;
            uint8_t *orow = (uint8_t *)p.out + ((size_t)m * p.N + n0 + cb) * esz;
#pragma unroll 1
            for (int c0 = 0; c0 < half; c0 += 32) {
                uint32_t v[32];
                mx_tmem_ld32(taddr + c0, v);              // (the load may run past the set's columns: those are not stored)
                if (!m_ok) continue;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int c = c0 + 8 * g;
                    if (n0 + cb + c >= p.N || c >= half) break;   // N and the set's width are multiples of 8
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[8 * g + j]);
                    if (p.out_type == ET_F32) {
                        float4 *o = reinterpret_cast<float4 *>(orow + (size_t)c * 4);
                        o[0] = make_float4(f[0], f[1], f[2], f[3]);
                        o[1] = make_float4(f[4], f[5], f[6], f[7]);
                    } else {
                        uint4 o;
                        if (p.out_type == ET_BF16) {
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(ab));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, MX_TMEM_COLS);
    }
}

// ---- preparation passes ---------------------------------------------------------------------------
// fp4 e2m1 codes (two per byte, element 0 = low nibble) -> the fp8 e4m3 byte of the same value.  A thread
// widens 16 packed bytes to 32.  Magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 are 0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48,
// 0x4C in e4m3; one byte-permute looks four of them up at once, the sign bit moves from bit 3 to bit 7.
__device__ __forceinline__ uint32_t fp4x4_to_e4m3x4(uint32_t codes16) {
    const uint32_t mag = __byte_perm(0x3C383000u, 0x4C484440u, codes16 & 0x7777u);
    const uint32_t s = codes16 & 0x8888u;
    return mag | ((s & 0x8u) << 4) | ((s & 0x80u) << 8) | ((s & 0x800u) << 12) | ((s & 0x8000u) << 16);
}
__global__ void __launch_bounds__(256) mx_widen_fp4_kernel(const uint4 *src, uint4 *dst, size_t n16) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n16) return;
    const uint4 v = __ldg(src + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        o[2 * j] = fp4x4_to_e4m3x4(w[j] & 0xFFFFu);
        o[2 * j + 1] = fp4x4_to_e4m3x4(w[j] >> 16);
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// Scales into 512-byte groups of 128 rows x 4 K blocks: byte (r % 32) * 16 + (r / 32) * 4 + block.
// along_rows: the source is [rows][kblocks] (operand A), groups ordered [row tile][k chunk]; otherwise the source is
// [kblocks][rows] (operand B: rows = output columns), groups ordered [k chunk][row tile], row tiles padded to `row_tiles`.
// Rows beyond the matrix get 127 (a scale of one; their elements are zero).  One CTA of 512 threads per group: the
// reads follow the source's contiguous direction, the re-ordering goes through shared memory, the writes are contiguous.
// Operand B's groups come in pairs per output tile: group 2 j + h covers the 128 columns from tile_n * j + 128 * h
// (tile_n = 256: plain consecutive groups).
__global__ void __launch_bounds__(512) mx_group_scales_kernel(const uint8_t *src, uint8_t *dst, int rows, int kblocks, int along_rows,
                                                              int row_tiles, int kchunks, int tile_n) {
    __shared__ uint8_t tile[4][128];   // [block][row]
    const int grp = blockIdx.x, t = threadIdx.x;
    const int rt = along_rows ? grp / kchunks : grp % row_tiles, kc = along_rows ? grp % kchunks : grp / row_tiles;
    {
        const int rl = along_rows ? t >> 2 : t & 127, kl = along_rows ? t & 3 : t >> 7;
        const int r = (along_rows ? rt * 128 : (rt >> 1) * tile_n + (rt & 1) * 128) + rl, kb = kc * 4 + kl;
        uint8_t v = 127;
        if (r < rows && kb < kblocks) v = along_rows ? src[(size_t)r * kblocks + kb] : src[(size_t)kb * rows + r];
        tile[kl][rl] = v;
    }
    __syncthreads();
    dst[(size_t)grp * 512 + t] = tile[t & 3][(t >> 4) + 32 * ((t >> 2) & 3)];
}

inline uint64_t mx_up256(uint64_t x) { return (x + 255) / 256 * 256; }

struct MxLayout {
    uint64_t a8, b8, sfa, sfb, total;
    int m_tiles, n_tiles, n128e, kchunks, tile_n, nacc, mh, a_groups;
};
int mx_sm_count() {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    return sms;
}
MxLayout mx_layout(const MatmulArgs &p) {
    MxLayout l{};
    // Tile shape.  What bounds the kernel is the operand traffic from L2 into shared memory -- (rows + columns) x K bytes per
    // tile, about 100 GB/s per SM -- not the tensor pipe (4096 x 8192 x 8192, one 128-row accumulator: 247 us at 256 columns,
    // 261 at 224, 311 at 192 even with a second accumulator hiding the epilogue, 411 at 128).  So with more than 256 rows a
    // tile is 256 rows x 224 columns: two accumulators (2 x 224 tensor-memory columns + the scales' 32) over ONE weight tile,
    // a third less traffic per output (4096 x 8192 x 8192: 249 -> 225 us; 245 us at 240 columns, 255 at 192), where that
    // does not leave SMs without a tile.  Otherwise 128 x 256 with one accumulator.
    // B200_QMM_MX_ROWS=128|256, B200_QMM_MX_TILE=<columns, a multiple of 16>, B200_QMM_MX_NACC=1 select other forms.
    {
        // rounds of one tile per SM x the measured time of a K block in either form (0.55 us at 128 x 256, 0.86 us at 256 x 224)
        const long long sms = mx_sm_count();
        const long long t1 = ((p.M + MX_M - 1) / MX_M) * ((p.N + MX_N - 1) / MX_N), t2 = ((p.M + 2 * MX_M - 1) / (2 * MX_M)) * ((p.N + 223) / 224);
        l.mh = p.M > 2 * MX_M && (double)((t2 + sms - 1) / sms) * 0.86 < (double)((t1 + sms - 1) / sms) * 0.55 ? 2 : 1;
    }
    if (const char *e = getenv("B200_QMM_MX_ROWS")) { const int v = atoi(e); if (v == 128) l.mh = 1; else if (v == 256) l.mh = 2; }
    l.tile_n = l.mh == 2 ? 224 : MX_N;
    if (const char *e = getenv("B200_QMM_MX_TILE")) { const int v = atoi(e); if (v >= 32 && v <= MX_N && v % 16 == 0) l.tile_n = v; }
    if (l.mh == 2 && 2 * l.tile_n > (int)MX_SF_COL) l.tile_n = 240;      // two row halves need two accumulators in front of the scales
    l.nacc = (l.mh == 1 && 2 * l.tile_n <= (int)MX_SF_COL) ? 2 : 1;
    if (const char *e = getenv("B200_QMM_MX_NACC")) { if (atoi(e) == 1) l.nacc = 1; }
    l.m_tiles = (int)((p.M + l.mh * MX_M - 1) / (l.mh * MX_M));
    l.a_groups = l.m_tiles * l.mh;                                      // 128-row scale groups of A
    l.n_tiles = (int)((p.N + l.tile_n - 1) / l.tile_n);
    l.n128e = 2 * l.n_tiles;
    l.kchunks = (int)(p.K / MX_BK);
    l.a8 = p.a_type == ET_E2M1 ? mx_up256((uint64_t)p.M * p.K) : 0;
    l.b8 = (p.b_type == ET_E2M1 && !p.b_nz) ? mx_up256((uint64_t)p.K * p.N) : 0;   // b_nz: widened once at load time
    l.sfa = mx_up256((uint64_t)l.a_groups * l.kchunks * 512);
    l.sfb = mx_up256((uint64_t)l.kchunks * l.n128e * 512);
    l.total = l.a8 + l.b8 + l.sfa + l.sfb;
    return l;
}

}  // namespace

bool mx_native_supported(const MatmulArgs &p) {
    if (p.epilogue != EPI_PLAIN || !p.a_scale || !p.b_scale || p.batch != 1 || p.b_transposed || p.accumulate || p.bias) return false;
    auto ok = [](int t) { return t == ET_E4M3 || t == ET_E5M2 || t == ET_E2M1; };
    if (!ok(p.a_type) || !ok(p.b_type)) return false;
    if (p.out_type != ET_BF16 && p.out_type != ET_F16 && p.out_type != ET_F32) return false;
    if (p.M < 1 || p.K < MX_BK || p.K % MX_BK != 0 || p.N % 32 != 0) return false;
    if (p.M > (1 << 24) || p.N > (1 << 24) || p.K > (1 << 24)) return false;
    if (const char *e = getenv("B200_QMM_MX_NATIVE")) {
        if (atoi(e) == 0) return false;
    }
    return true;
}

uint64_t mx_native_workspace_bytes(const MatmulArgs &p) { return mx_layout(p).total; }

cudaError_t launch_mx_native(const MatmulArgs &p, cudaStream_t s) {
    const MxLayout l = mx_layout(p);
    if (!p.workspace || p.workspace_bytes < l.total) return cudaErrorInvalidValue;
    auto misaligned16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
    if (misaligned16(p.a) || misaligned16(p.b) || misaligned16(p.out) || misaligned16(p.workspace)) return cudaErrorMisalignedAddress;
    uint8_t *ws = (uint8_t *)p.workspace;
    uint8_t *a8 = ws, *b8 = ws + l.a8, *sfa = b8 + l.b8, *sfb = sfa + l.sfa;
    const uint8_t *a_src = (const uint8_t *)p.a, *b_src = (const uint8_t *)p.b;
    if (p.a_type == ET_E2M1) {
        const size_t n16 = (size_t)p.M * p.K / 32;   // 16 packed bytes = 32 elements; K % 128 == 0
        mx_widen_fp4_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, s>>>((const uint4 *)p.a, (uint4 *)a8, n16);
        count_launch();
        a_src = a8;
    }
    if (p.b_type == ET_E2M1 && !p.b_nz) {
        const size_t n16 = (size_t)p.K * p.N / 32;   // N % 32 == 0
        mx_widen_fp4_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, s>>>((const uint4 *)p.b, (uint4 *)b8, n16);
        count_launch();
        b_src = b8;
    }
    const int kblocks = (int)(p.K / 32);
    {
        mx_group_scales_kernel<<<(unsigned)(l.a_groups * l.kchunks), 512, 0, s>>>(p.a_scale, sfa, (int)p.M, kblocks, 1, l.a_groups, l.kchunks, 128);
        mx_group_scales_kernel<<<(unsigned)(l.kchunks * l.n128e), 512, 0, s>>>(p.b_scale, sfb, (int)p.N, kblocks, 0, l.n128e, l.kchunks, l.tile_n);
        count_launch(2);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;

    CUtensorMap ta, tb;
    // With several row tiles the CTAs that share a weight tile run together: keep the wider L2 fetch.
    bool ok = make_map(&ta, a_src, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.K, p.M, p.K, 128, MX_M, CU_TENSOR_MAP_SWIZZLE_128B) &&
              make_map(&tb, b_src, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.N, p.K, p.N, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorInvalidValue;

    MxParams mp{};
    mp.out = p.out; mp.out_type = p.out_type;
    mp.M = (int)p.M; mp.N = (int)p.N; mp.K = (int)p.K;
    mp.m_tiles = l.m_tiles; mp.tiles = l.m_tiles * l.n_tiles; mp.num_kb = l.kchunks;
    mp.sfa = sfa; mp.sfb = sfb; mp.n128e = l.n128e; mp.tile_n = l.tile_n; mp.nacc = l.nacc;
    const int a_fmt = p.a_type == ET_E5M2 ? 1 : 0, b_fmt = p.b_type == ET_E5M2 ? 1 : 0;   // widened fp4 is e4m3
    const uint32_t idesc = mx_idesc(a_fmt, b_fmt, MX_M, l.tile_n);

    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        e = cudaFuncSetAttribute(mx_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<1>::TOTAL);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(mx_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<2>::TOTAL);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    const int sms = mx_sm_count();
    const int P = mp.tiles < sms ? mp.tiles : sms;
    if (l.mh == 2) mx_tc_kernel<2><<<P, 320, MxSmem<2>::TOTAL, s>>>(ta, tb, mp, idesc);
    else mx_tc_kernel<1><<<P, 320, MxSmem<1>::TOTAL, s>>>(ta, tb, mp, idesc);
    count_launch();
    return cudaGetLastError();
}

// One-time widening of an fp4 weight [K,N] to its e4m3 bytes (the on-device format of fp4 weights: K * N bytes).
cudaError_t launch_mx_widen_fp4(const void *src, void *dst, int64_t elems, cudaStream_t s) {
    if (elems % 32 != 0) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return cudaErrorMisalignedAddress;
    const size_t n16 = (size_t)elems / 32;
    mx_widen_fp4_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, s>>>((const uint4 *)src, (uint4 *)dst, n16);
    count_launch();
    return cudaGetLastError();
}

unsigned int mx_tc_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    return v;
}
void mx_tc_device_status_reset() {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(z));
}

}  // namespace qmm
