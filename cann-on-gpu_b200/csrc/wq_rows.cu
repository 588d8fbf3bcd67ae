// W4A16 / W8A16 decode kernel for 3 to 16 rows: TMA-staged packed weights in the caller's [K,N] layout, dequantised in
// registers, multiplied on the warp-level tensor-core path (mma.sync m16n8k16) in the activation type, group scales
// folded in fp32, stream-K.  (One and two rows, and every row count on tile-packed weights, run wq_mma.cu, which
// converts the activations to fp16 inside the kernel; with more rows that conversion does not keep up and this
// kernel, which feeds the activations to the tensor core as they are, is the faster one.)
//
// Per CTA (one per SM, 14 warps):
//   warp 0       producer: one TMA per super-block (128 K rows x 256 columns of packed int4 = 16 KB,
//                128-byte swizzle, no L2 promotion) plus the activation rows of the same K range, into
//                a ring of two to four slots per team (as many as fit beside the partial tiles).
//   warps 1-12   three teams of four warps.  A team owns one quantum (= one scale group, or one
//                super-block for per-channel scales) at a time; each of its warps covers 64 of the
//                tile's 256 columns.  Per 16 K rows a lane reads four 32-bit words (rows 2t, 2t+1,
//                2t+8, 2t+9 of its 8 columns -- bank-conflict free under the swizzle), interleaves row
//                pairs with two byte-permutes and extracts each (k, k+1) nibble pair with one lop3
//                into a bf16x2 / fp16x2 register holding the exact integers 136+q / 1032+q; these are
//                the A fragments (weights^T) of mma.sync, the activations are the B fragments, and
//                one more mma with an all-ones A accumulates the activation sums.  At the end of the
//                group:   tot += s_g[n] * (acc - (136 + off_g[n]) * sum_g x)
//                which is the reference's algebra (cuda/src/ops/matmul.cu:334-335) per group, in fp32.
//   warp 13      reducer: when all teams have finished a tile (or this CTA's piece of it) it sums the
//                teams' partial tiles from shared memory in a fixed order and writes the output
//                (whole tile) or an fp32 slot (piece; summed by wq_rows_finalize_kernel).
// Work split: the (tile, quantum) space is cut into gridDim.x equal contiguous shares (stream-K).
// Every ring slot belongs to one team, so a team meets the phases of a slot's barrier in order and a
// parity wait can never be asked about a phase that is two ahead.
//
// int8 weights use the same path: a byte is lo + 16 * hi (unsigned low nibble, signed high nibble); the
// two nibbles ride rows g and g+8 of one mma and are recombined in the fold (tile = 128 columns).
//
// Replaces the reference's k_wq_fused (cuda/src/ops/matmul.cu:337-352).
#include <mutex>
#include <type_traits>

#include "tc_common.cuh"

namespace qmm {
namespace {

constexpr int MM_TILE_N = 256;      // output columns per tile
constexpr int MM_SBK = 128;         // K rows per super-block (the unit scale groups are counted in)
constexpr int MM_W_BYTES = 16384;   // packed weights of one super-block: 128 rows x 128 B

struct MmParams {
    void *out;
    float *slots;            // [tiles + P][M][tile_n] fp32 partial tiles
    const void *scale, *offset, *bias;
    int sc_type, out_type;
    int M, N, K;
    int sbq;                 // super-blocks per quantum
    int qpt;                 // quanta per tile
    long long total_q;       // tiles * qpt
    int grouped;
    int ns;                  // ring slots (a multiple of the team count, see mm_ring_slots)
    int tile_n;              // output columns per tile: 256 (int4) or 128 (int8: two nibbles per column)
};

// Shared memory of one CTA: [ring: ns slots][partial tiles: teams x M rows x 256 fp32][barriers][flag].
template <int MF>
struct MmSmem {
    static constexpr int XBOX = MF * 8 * 128;                 // one activation box: MF*8 rows x 64 k
    static constexpr int SLOT = MM_W_BYTES + 2 * XBOX;        // multiple of 1024
    __host__ __device__ static int part_bytes(int teams, int M) { return teams * M * MM_TILE_N * 4; }   // sized for the wider (int4) tile
    __host__ __device__ static int bar_off(int ns, int teams, int M) { return ns * SLOT + part_bytes(teams, M); }
    __host__ __device__ static int total(int ns, int teams, int M) { return bar_off(ns, teams, M) + (2 * ns + 2) * 8 + 16 + 1024; }
};

__host__ __device__ inline long long mm_share_begin(long long c, long long total_q, int P) { return c * total_q / P; }
__host__ __device__ inline int mm_share_owner(long long q, long long total_q, int P) { return (int)(((q + 1) * P - 1) / total_q); }

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// The same with a zero C operand: the first step of a group needs no cleared accumulators.
template <bool BF16>
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
    }
}

// Two nibbles (bits 0-3 and 16-19) -> two 16-bit floats holding the integers MAGIC + q, q the signed
// 4-bit value: xor 8 turns the two's-complement nibble into q + 8 in the low mantissa bits of
// 128.0 (bf16) or 1024.0 (fp16).  One lop3, (v & mask) ^ magic, with both constants in registers.
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
template <bool BF16> __device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    if constexpr (BF16) return __uint_as_float(h << 16);
    return __half2float(__ushort_as_half((unsigned short)h));
}

__device__ __forceinline__ uint2 ldg8_now(const void *ptr) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
    return v;
}

// Bounded wait that ignores the abort flag (used only to let copies in flight land before exit).
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (global_ns() - t0 > 2000000ull) return;
    }
}

template <bool Q8, bool BF16, int MF, int MM_TEAMS>
__global__ void __launch_bounds__((4 * MM_TEAMS + 2) * 32, 1)
wq_rows_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const MmParams p) {
    using L = MmSmem<MF>;
    constexpr int TN = Q8 ? 128 : 256;   // output columns per tile (the tile is 256 nibble columns wide)
    const int MM_NS = p.ns;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    const int bar_off = L::bar_off(MM_NS, MM_TEAMS, p.M);
    const uint32_t bars = base + bar_off;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (MM_NS + s); };
    const uint32_t seg_done = bars + 8u * (2 * MM_NS), seg_free = bars + 8u * (2 * MM_NS + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + bar_off + (2 * MM_NS + 2) * 8);
    float *part = reinterpret_cast<float *>(gen_base + MM_NS * L::SLOT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int P = gridDim.x, cta = blockIdx.x;
    const long long qb = mm_share_begin(cta, p.total_q, P), qe = mm_share_begin(cta + 1, p.total_q, P);
    const int nq = (int)(qe - qb);
    const int tile_first = (int)(qb / p.qpt), tile_last = (int)((qe - 1) / p.qpt);

    if (threadIdx.x == 0) {
        for (int s = 0; s < MM_NS; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 4); }
        mbar_init(seg_done, 4 * MM_TEAMS);
        mbar_init(seg_free, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int i = 0, slot = 0, round = 0;
            int tile = tile_first, qi = (int)(qb - (long long)tile_first * p.qpt);
            bool ok = true;
            for (int j = 0; j < nq && ok; ++j) {
                for (int u = 0; u < p.sbq; ++u, ++i) {
                    const int k0 = (qi * p.sbq + u) * MM_SBK;
                    if (round > 0 && !mbar_wait(empty_bar(slot), (round - 1) & 1, abort_flag, 0x300u + slot)) { ok = false; break; }
                    const uint32_t dst = base + slot * L::SLOT;
                    mbar_expect_tx(full_bar(slot), L::SLOT);
                    tma_load_2d(dst, &tm_w, full_bar(slot), tile * 128, k0);
                    tma_load_2d(dst + MM_W_BYTES, &tm_x, full_bar(slot), k0, 0);
                    tma_load_2d(dst + MM_W_BYTES + L::XBOX, &tm_x, full_bar(slot), k0 + 64, 0);
                    if (++slot == MM_NS) { slot = 0; ++round; }
                }
                if (++qi == p.qpt) { qi = 0; ++tile; }
            }
            if (!ok) {   // let the copies already issued land before the CTA's shared memory goes away
                for (int b = (i > MM_NS ? i - MM_NS : 0); b < i; ++b) mbar_drain(full_bar(b % MM_NS), (b / MM_NS) & 1);
            }
        }
    } else if (warp <= 4 * MM_TEAMS) {
        // ------------------------------------------------------------------ compute
        const int cw = warp - 1, team = cw >> 2, wq = cw & 3;
        const int g = lane >> 2, t = lane & 3;
        // byte offsets inside a slot of the four weight words of step 0 (rows 2t, 2t+1, 2t+8, 2t+9)
        uint32_t woff[4];
        {
            const int c16 = 2 * wq + (g >> 2), inb = 4 * (g & 3);
            const int rows[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
            for (int j = 0; j < 4; ++j) woff[j] = 128 * rows[j] + (((c16 ^ (rows[j] & 7)) << 4)) + inb;
        }
        // activation words: slot + xrow, with the 16-byte chunk index xor-ed in (the swizzle); + box,
        // + 1024 for the second fragment
        const uint32_t xrow = MM_W_BYTES + 128 * g + 16 * g + 4 * t;
        constexpr uint32_t ONES = BF16 ? 0x3F803F80u : 0x3C003C00u;
        // int4: every nibble is a signed weight (xor 8 -> q + 8 above 128.0 / 1024.0).  int8: the byte
        // is q = lo + 16 * hi with lo the unsigned low nibble (no xor) and hi the signed high nibble.
        uint32_t dq_mask = 0x000F000Fu, dq_magic = BF16 ? 0x43084308u : 0x64086408u;
        uint32_t dq_magic_even = Q8 ? (BF16 ? 0x43004300u : 0x64006400u) : dq_magic;
        uint32_t dq_mask2 = 0x00F000F0u, dq_magic2 = 0x64806480u;   // fp16 only: nibble at bits 4-7
        asm volatile("" : "+r"(dq_mask), "+r"(dq_magic), "+r"(dq_magic_even), "+r"(dq_mask2), "+r"(dq_magic2));   // keep the constants in registers
        constexpr float MAGIC = BF16 ? 136.f : 1032.f;
        // first of this lane's columns inside the tile: 8 nibble columns = 8 (int4) or 4 (int8) outputs
        const int n_lane = Q8 ? 32 * wq + 4 * g : 64 * wq + 8 * g;

        float acc[MF][4][4], tot[MF][4][4], xs[MF][4];
        bool ok = true;
        int sg = 0;
        // This team's stages are i = j * sbq + u for its quanta j = team, team + TEAMS, ...; their ring
        // slot and pass number are kept incrementally.
        int slot = team * p.sbq, round = 0;
        for (int tile = tile_first; tile <= tile_last && ok; ++tile, ++sg) {
            const long long t_lo = (long long)tile * p.qpt, t_hi = t_lo + p.qpt;
            const int j_lo = (int)((t_lo > qb ? t_lo : qb) - qb), j_hi = (int)((t_hi < qe ? t_hi : qe) - qb);
            const int n_glob = tile * TN + n_lane;
            const bool n_ok = n_glob < p.N;
            bool had = false;
#pragma unroll
            for (int f = 0; f < MF; ++f)
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int e = 0; e < 4; ++e) tot[f][r][e] = 0.f;
            // scale / offset rows of a group: 8 consecutive columns = 16 bytes per lane (8 bytes for int8
            // weights), fetched one quantum ahead of their use.  Lanes beyond N read column 0 (unused).
            const int n_safe = n_ok ? n_glob : 0;
            const int qi_seg = (int)(qb + j_lo - t_lo);   // quantum index inside the tile of local quantum j_lo
            const int j_first = j_lo + (team - j_lo % MM_TEAMS + MM_TEAMS) % MM_TEAMS;
            const size_t row_step = p.grouped ? (size_t)MM_TEAMS * p.N : 0;
            const uint16_t *sc_ptr = static_cast<const uint16_t *>(p.scale) + n_safe +
                                     (p.grouped ? (size_t)(qi_seg + j_first - j_lo) * p.N : 0);
            const uint16_t *of_base = p.offset ? static_cast<const uint16_t *>(p.offset) : nullptr;
            const ptrdiff_t of_delta = of_base ? reinterpret_cast<const uint16_t *>(p.offset) - reinterpret_cast<const uint16_t *>(p.scale) : 0;
            auto fetch_rows = [&](const uint16_t *sp, uint4 &sr, uint4 &orr) {
                if constexpr (Q8) {
                    const uint2 a = ldg8_now(sp);
                    sr.x = a.x; sr.y = a.y;
                    if (of_base) { const uint2 b = ldg8_now(sp + of_delta); orr.x = b.x; orr.y = b.y; }
                } else {
                    sr = ldg16_now(sp);
                    if (of_base) orr = ldg16_now(sp + of_delta);
                }
            };
            uint4 sraw = make_uint4(0, 0, 0, 0), oraw = sraw, snext = sraw, onext = sraw;
            if (j_first < j_hi) fetch_rows(sc_ptr, snext, onext);
            for (int j = j_first; j < j_hi && ok; j += MM_TEAMS) {
                had = true;
                sraw = snext;
                oraw = onext;
                if (j + MM_TEAMS < j_hi) sc_ptr += row_step;   // the last quantum fetches its own row again
                fetch_rows(sc_ptr, snext, onext);
                for (int u = 0; u < p.sbq && ok; ++u) {
                    const bool first_sb = u == 0;
                    if (!mbar_wait(full_bar(slot), round & 1, abort_flag, 0x310u + slot)) { ok = false; break; }
                    const uint32_t sb = base + slot * L::SLOT, xb = sb + xrow;
#pragma unroll
                    for (int st = 0; st < 8; ++st) {
                        const uint32_t w0 = lds32(sb + woff[0] + st * 2048), w1 = lds32(sb + woff[1] + st * 2048);
                        const uint32_t w2 = lds32(sb + woff[2] + st * 2048), w3 = lds32(sb + woff[3] + st * 2048);
                        uint32_t b0[MF], b1[MF];
                        {
                            const uint32_t xa0 = xb ^ ((uint32_t)(2 * (st & 3)) << 4), xa1 = xb ^ ((uint32_t)(2 * (st & 3) + 1) << 4);
#pragma unroll
                            for (int f = 0; f < MF; ++f) {
                                b0[f] = lds32(xa0 + (st >> 2) * L::XBOX + f * 1024);
                                b1[f] = lds32(xa1 + (st >> 2) * L::XBOX + f * 1024);
                            }
                        }
                        // rows (k, k+1) side by side: low halves = nibbles 0-3, high halves = nibbles 4-7
                        const uint32_t lo[2] = {__byte_perm(w0, w1, 0x5410), __byte_perm(w0, w1, 0x7632)};
                        const uint32_t hi[2] = {__byte_perm(w2, w3, 0x5410), __byte_perm(w2, w3, 0x7632)};
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int sh = (r & 1) * 8;
                            uint32_t a0, a1, a2, a3;
                            if constexpr (BF16) {
                                a0 = dq_pair(lo[r >> 1] >> sh, dq_mask, dq_magic_even);
                                a1 = dq_pair(lo[r >> 1] >> (sh + 4), dq_mask, dq_magic);
                                a2 = dq_pair(hi[r >> 1] >> sh, dq_mask, dq_magic_even);
                                a3 = dq_pair(hi[r >> 1] >> (sh + 4), dq_mask, dq_magic);
                            } else {
                                // fp16 has room for a nibble at mantissa bits 4-7 too: the odd column of
                                // each pair is taken in place as 1152 + 16 q (undone in the fold), which
                                // saves its shift
                                const uint32_t l = lo[r >> 1] >> sh, h = hi[r >> 1] >> sh;
                                a0 = dq_pair(l, dq_mask, dq_magic_even);
                                a1 = dq_pair(l, dq_mask2, dq_magic2);
                                a2 = dq_pair(h, dq_mask, dq_magic_even);
                                a3 = dq_pair(h, dq_mask2, dq_magic2);
                            }
#pragma unroll
                            for (int f = 0; f < MF; ++f) {
                                if (st == 0 && first_sb) mma16816_first<BF16>(acc[f][r], a0, a1, a2, a3, b0[f], b1[f]);
                                else mma16816<BF16>(acc[f][r], a0, a1, a2, a3, b0[f], b1[f]);
                            }
                        }
#pragma unroll
                        for (int f = 0; f < MF; ++f) {
                            if (st == 0 && first_sb) mma16816_first<BF16>(xs[f], ONES, ONES, ONES, ONES, b0[f], b1[f]);
                            else mma16816<BF16>(xs[f], ONES, ONES, ONES, ONES, b0[f], b1[f]);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar(slot));
                    if (++slot == MM_NS) { slot = 0; ++round; }
                }
                // skip the other teams' stages of this round robin
                slot += (MM_TEAMS - 1) * p.sbq;
                while (slot >= MM_NS) { slot -= MM_NS; ++round; }
                // fold the finished group (one uniform branch on the presence of offsets, so that the
                // common offset-free form carries no conversions or selects for them)
                const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w}, ow[4] = {oraw.x, oraw.y, oraw.z, oraw.w};
                auto fold = [&](auto has_off) {
                    constexpr bool OFF = decltype(has_off)::value;
                    if constexpr (Q8) {
                        // column r of this lane: rows g (low nibbles, MAGIC_LO + lo) and g+8 (high nibbles,
                        // bf16: 136 + hi, to be taken 16 times; fp16: 1152 + 16 hi) of the same mma
                        constexpr float HM = BF16 ? 16.f : 1.f, C = BF16 ? 128.f + 16.f * 136.f : 1024.f + 1152.f;
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const float sn = half_bits_to_float<BF16>((r & 1) ? sw[r >> 1] >> 16 : sw[r >> 1] & 0xFFFFu);
                            float cn = C;
                            if constexpr (OFF) cn += half_bits_to_float<BF16>((r & 1) ? ow[r >> 1] >> 16 : ow[r >> 1] & 0xFFFFu);
#pragma unroll
                            for (int f = 0; f < MF; ++f)
#pragma unroll
                                for (int e = 0; e < 2; ++e)
                                    tot[f][r][e] = fmaf(sn, fmaf(-cn, xs[f][e], fmaf(HM, acc[f][r][2 + e], acc[f][r][e])), tot[f][r][e]);
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                float sn = half_bits_to_float<BF16>(h ? sw[r] >> 16 : sw[r] & 0xFFFFu);
                                // odd columns of the fp16 form were accumulated as 1152 + 16 q
                                const bool scaled = !BF16 && h;
                                float cn = scaled ? 1152.f : MAGIC;
                                if constexpr (OFF) {
                                    const float off = half_bits_to_float<BF16>(h ? ow[r] >> 16 : ow[r] & 0xFFFFu);
                                    cn += scaled ? 16.f * off : off;
                                }
                                if (scaled) sn *= 0.0625f;
#pragma unroll
                                for (int f = 0; f < MF; ++f)
#pragma unroll
                                    for (int e = 0; e < 2; ++e)
                                        tot[f][r][2 * h + e] = fmaf(sn, fmaf(-cn, xs[f][e], acc[f][r][2 * h + e]), tot[f][r][2 * h + e]);
                            }
                        }
                    }
                };
                if (of_base) fold(std::true_type{});
                else fold(std::false_type{});
            }
            if (!ok) break;
            // hand this team's partial tile to the reducer
            if (sg >= 1 && !mbar_wait(seg_free, (sg - 1) & 1, abort_flag, 0x320u)) { ok = false; break; }
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
            const long long t_lo = (long long)tile * p.qpt, t_hi = t_lo + p.qpt;
            const int j_lo = (int)((t_lo > qb ? t_lo : qb) - qb), j_hi = (int)((t_hi < qe ? t_hi : qe) - qb);
            const int cnt = j_hi - j_lo;
            const bool whole = cnt == p.qpt;
            if (!mbar_wait(seg_done, sg & 1, abort_flag, 0x330u)) break;
            // each lane owns CPL consecutive columns
            constexpr int CPL = TN / 32;
            const int n = CPL * lane, n_glob = tile * TN + n;
            if (n_glob < p.N) {
                for (int m = 0; m < p.M; ++m) {
                    float v[CPL];
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
                    if (whole) {
                        uint32_t o[CPL / 2];
#pragma unroll
                        for (int c = 0; c < CPL / 2; ++c) {
                            float lo = v[2 * c], hi = v[2 * c + 1];
                            if (p.bias) {
                                lo += load_as_float(p.bias, p.sc_type, n_glob + 2 * c);
                                hi += load_as_float(p.bias, p.sc_type, n_glob + 2 * c + 1);
                            }
                            if constexpr (BF16) {
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi);
                                o[c] = *reinterpret_cast<uint32_t *>(&t2);
                            } else {
                                __half2 t2 = __floats2half2_rn(lo, hi);
                                o[c] = *reinterpret_cast<uint32_t *>(&t2);
                            }
                        }
                        uint16_t *dst = static_cast<uint16_t *>(p.out) + (size_t)m * p.N + n_glob;
                        if constexpr (Q8) *reinterpret_cast<uint2 *>(dst) = make_uint2(o[0], o[1]);
                        else *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
                    } else {
                        float4 *dst = reinterpret_cast<float4 *>(p.slots + ((size_t)(tile + cta) * p.M + m) * TN + n);
#pragma unroll
                        for (int c = 0; c < CPL / 4; ++c) dst[c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(seg_free);
        }
    }
}

// Sums the partial tiles of every output tile that was shared between CTAs, adds the bias, casts.
__global__ void wq_rows_finalize_kernel(MmParams p, int P) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)p.M * p.N) return;
    const int n = (int)(i % p.N), m = (int)(i / p.N);
    const int tile = n / p.tile_n;
    const long long qa = (long long)tile * p.qpt;
    const int c_first = mm_share_owner(qa, p.total_q, P), c_last = mm_share_owner(qa + p.qpt - 1, p.total_q, P);
    if (c_first == c_last) return;  // written directly by its only owner
    float v = 0.f;
    for (int c = c_first; c <= c_last; ++c) v += p.slots[((size_t)(tile + c) * p.M + m) * p.tile_n + (n % p.tile_n)];
    if (p.bias) v += load_as_float(p.bias, p.sc_type, n);
    store_from_float(p.out, p.out_type, i, v);
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
    int mf, tiles, sbq, qpt, grouped, P;
    long long total_q;
    uint64_t slot_bytes;
};

MmPlan mm_make_plan(const MatmulArgs &p) {
    MmPlan pl{};
    pl.mf = p.M <= 8 ? 1 : 2;
    const int tile_n = p.b_type == ET_I8 ? 128 : 256;
    pl.tiles = (int)((p.N + tile_n - 1) / tile_n);
    const int num_sb = (int)((p.K + MM_SBK - 1) / MM_SBK);
    pl.grouped = p.group < p.K ? 1 : 0;
    pl.sbq = pl.grouped ? (int)(p.group / MM_SBK) : 1;
    pl.qpt = num_sb / pl.sbq;
    pl.total_q = (long long)pl.tiles * pl.qpt;
    const int sms = mm_sm_count();
    pl.P = (int)(pl.total_q < sms ? pl.total_q : sms);
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
    // multiple) of a tile's quanta, so each CTA adds to one tile only and fewer partial tiles are written and
    // summed (4096 x 4096 int4 at M = 16: 16.7 us on 148 CTAs, 14.9 us on 128).  Take the largest such CTA
    // count within 15 % of the SM count.  B200_QMM_WQ_MMA_P=<n> overrides.
    if (pl.P == sms && pl.total_q < 8LL * sms) {   // small problems only: large ones are bound by the work per SM
        for (int c = sms; c >= sms - sms * 15 / 100; --c) {
            if (pl.total_q % c != 0) continue;
            const long long share = pl.total_q / c;
            if (pl.qpt % share == 0 || share % pl.qpt == 0) { pl.P = c; break; }
        }
    }
    if (const char *e = getenv("B200_QMM_WQ_MMA_P")) { const int v = atoi(e); if (v >= 1 && v <= sms && v <= pl.total_q) pl.P = v; }
    pl.slot_bytes = (uint64_t)(pl.tiles + pl.P) * p.M * tile_n * sizeof(float);
    return pl;
}

constexpr int MM_TEAMS_USED = 3;
constexpr int MM_SMEM_LIMIT = 232448;

// Ring depth: every slot must belong to one team (a team then meets the phases of a slot's barrier in
// order), so the depth is c x teams, and with two super-blocks per quantum c must be even.  Three or
// four slots per team hide the HBM round trip (one being read, the others in flight); take the
// deepest ring that fits beside the partial tiles.
template <int MF>
int mm_ring_slots(int M, int sbq) {
    for (int c = 4; c >= 2; --c) {
        if (sbq == 2 && (c & 1)) continue;
        if (MmSmem<MF>::total(c * MM_TEAMS_USED, MM_TEAMS_USED, M) <= MM_SMEM_LIMIT) return c * MM_TEAMS_USED;
    }
    return 0;
}

template <bool Q8, bool BF16, int MF>
cudaError_t mm_launch_one(const CUtensorMap &tx, const CUtensorMap &tw, MmParams mp, int P, cudaStream_t s) {
    using L = MmSmem<MF>;
    static_assert(L::SLOT % 1024 == 0, "slots keep the swizzle alignment");
    mp.ns = mm_ring_slots<MF>(mp.M, mp.sbq);
    if (mp.ns == 0) return cudaErrorInvalidValue;
    const int smem = L::total(mp.ns, MM_TEAMS_USED, mp.M);
    auto kern = wq_rows_kernel<Q8, BF16, MF, MM_TEAMS_USED>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_set[dev & 63] = true;
    }
    kern<<<P, (4 * MM_TEAMS_USED + 2) * 32, smem, s>>>(tx, tw, mp);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

bool wq_rows_supported(const MatmulArgs &p) {
    if (p.epilogue != EPI_PLAIN || !p.scale || p.a_scale || p.b_scale) return false;
    if (p.batch != 1 || p.b_transposed || p.b_nz || p.accumulate || p.M < 1 || p.M > 16) return false;
    if (p.a_type != ET_F16 && p.a_type != ET_BF16) return false;
    if (p.b_type != ET_I4 && p.b_type != ET_I8) return false;
    if (p.sc_type != p.a_type || p.out_type != p.a_type || (p.bias && p.bias_type != p.a_type)) return false;
    if (p.K % 8 != 0 || p.K < MM_SBK || p.N % (p.b_type == ET_I4 ? 32 : 16) != 0) return false;
    if (p.group < p.K) {
        if (p.group % MM_SBK != 0 || p.K % p.group != 0) return false;
        // a ring slot must belong to one team: the ring is two quanta per team deep
        if (p.group / MM_SBK > 2) return false;
    }
    if (p.N > (1 << 24) || p.K > (1 << 24)) return false;
    return true;
}

uint64_t wq_rows_workspace_bytes(const MatmulArgs &p) { return mm_make_plan(p).slot_bytes; }

cudaError_t launch_wq_rows(const MatmulArgs &p, cudaStream_t s) {
    const MmPlan pl = mm_make_plan(p);
    if (p.workspace_bytes < pl.slot_bytes || !p.workspace) return cudaErrorInvalidValue;
    // TMA sources, the 16-byte scale / offset loads, the 16-byte output stores and the float4 partial
    // tiles all need 16-byte aligned bases (every row pitch already is a multiple of 16 bytes).
    if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15) ||
        (reinterpret_cast<uintptr_t>(p.scale) & 15) || (reinterpret_cast<uintptr_t>(p.offset) & 15) ||
        (reinterpret_cast<uintptr_t>(p.out) & 15) || (reinterpret_cast<uintptr_t>(p.workspace) & 15))
        return cudaErrorMisalignedAddress;
    const bool bf = p.a_type == ET_BF16;
    CUtensorMap tx, tw;
    // No L2 promotion: every byte of the weight stream is used exactly once by exactly one CTA, and
    // fetching wider L2 lines than asked for measurably slows the stream down.
    bool ok = make_map(&tx, p.a, bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.K, p.M, p.K * 2, 64,
                       pl.mf * 8, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE);
    const bool q8 = p.b_type == ET_I8;
    const uint64_t row_bytes = q8 ? (uint64_t)p.N : (uint64_t)p.N / 2;
    ok = ok && make_map(&tw, p.b, CU_TENSOR_MAP_DATA_TYPE_UINT8, row_bytes, p.K, row_bytes, 128, MM_SBK, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE);
    if (!ok) return cudaErrorInvalidValue;

    MmParams mp{};
    mp.out = p.out;
    mp.slots = (float *)p.workspace;
    mp.scale = p.scale; mp.offset = p.offset; mp.bias = p.bias;
    mp.sc_type = p.sc_type; mp.out_type = p.out_type;
    mp.M = (int)p.M; mp.N = (int)p.N; mp.K = (int)p.K;
    mp.sbq = pl.sbq; mp.qpt = pl.qpt; mp.total_q = pl.total_q; mp.grouped = pl.grouped;
    mp.tile_n = q8 ? 128 : 256;

    cudaError_t e;
    if (q8) {
        if (pl.mf == 1) e = bf ? mm_launch_one<true, true, 1>(tx, tw, mp, pl.P, s) : mm_launch_one<true, false, 1>(tx, tw, mp, pl.P, s);
        else e = bf ? mm_launch_one<true, true, 2>(tx, tw, mp, pl.P, s) : mm_launch_one<true, false, 2>(tx, tw, mp, pl.P, s);
    } else {
        if (pl.mf == 1) e = bf ? mm_launch_one<false, true, 1>(tx, tw, mp, pl.P, s) : mm_launch_one<false, false, 1>(tx, tw, mp, pl.P, s);
        else e = bf ? mm_launch_one<false, true, 2>(tx, tw, mp, pl.P, s) : mm_launch_one<false, false, 2>(tx, tw, mp, pl.P, s);
    }
    if (e != cudaSuccess) return e;
    // Tiles shared between CTAs exist unless every share boundary falls on a tile boundary.
    if (pl.total_q % pl.P != 0 || (pl.total_q / pl.P) % pl.qpt != 0) {
        const size_t mn = (size_t)p.M * p.N;
        wq_rows_finalize_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(mp, pl.P);
        count_launch();
        e = cudaGetLastError();
    }
    return e;
}

void wq_rows_device_status_reset() {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(z));
}

unsigned int wq_rows_device_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    return v;
}

}  // namespace qmm
