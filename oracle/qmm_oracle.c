/*
 * qmm_oracle.c -- CPU restatement of the reference's quantized-matmul algorithms.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing on the product path links, loads or calls this file: it is
 * the checker used by tests/, by the smoke test and by the bench's cpu_baseline leg.
 *
 * Each function restates, as plain scalar loops, what the reference computes for one operator.
 * The reference has two statements of every algorithm: CUDA kernels (cuda/src/ops/matmul.cu) and
 * plain host loops in its Metal backend (metal/src/ops/conv.mm); both are cited per function.
 * Accumulation is in double (the Metal loops and the reference's own in-test CPU references do
 * the same: tests/test_matmul_conv.cpp:621-656), integer paths accumulate exactly in int64.
 *
 * Pinning: the reference stores no golden files for this path.  What it does hold -- the INT4-pack
 * known answer (tests/test_matmul_conv.cpp:938-945), the fp4 e2m1 decode table and encode
 * boundaries (cuda/src/ops/subfp.cuh:18-20,44; tests/test_fp8.cpp:149-191), e8m0 = 2^(e-127)
 * (tests/test_matmul_conv.cpp:247,309) and the in-test CPU references with their seeds and
 * tolerances -- is checked in tests/test_oracle.py.
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off -shared -fPIC)
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

/* ---------------------------------------------------------------- scalar codecs */

/* int4 element `idx` of a packed buffer: even linear index = low nibble, two's complement
 * (cuda/src/ops/matmul.cu:345-346,744; metal/src/ops/conv.mm K_WQMM rd_i4). */
static inline int int4_at(const uint8_t *p, int64_t idx) {
    uint8_t byte = p[idx >> 1];
    int v = (idx & 1) ? (byte >> 4) : (byte & 0xf);
    return v >= 8 ? v - 16 : v;
}

/* fp4 e2m1 magnitude table {0,.5,1,1.5,2,3,4,6}, sign in bit 3 (cuda/src/ops/subfp.cuh:18-20). */
static const float kE2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
EXPORT float oracle_e2m1_decode(uint8_t code) {
    float m = kE2M1[code & 7];
    return (code & 8) ? -m : m;
}

/* fp4 e2m1 encode: smallest |x| that selects magnitude code c (cuda/src/ops/subfp.cuh:44,62-70).
 * The sub-1.0 boundaries are the Ascend library's, not IEEE round-to-nearest-even; NaN -> 0;
 * out-of-range saturates to +-6. */
static const float kE2M1Bound[8] = {0.f, 0.4375f, 0.875f, 1.25000012f, 1.75f, 2.50000024f, 3.5f, 5.00000048f};
EXPORT uint8_t oracle_e2m1_encode(float x) {
    uint32_t xb; memcpy(&xb, &x, 4);
    if ((xb & 0x7fffffffu) > 0x7f800000u) return 0;
    float ax = fabsf(x);
    int c = 0;
    for (int i = 1; i < 8; i++) { if (ax >= kE2M1Bound[i]) c = i; else break; }
    return (uint8_t)((xb >> 31) ? (c | 8) : c);
}

/* fp8 decode: e4m3fn (bias 7, no inf, 0x7f/0xff = NaN) and e5m2 (IEEE-like, bias 15); what a cast
 * of __nv_fp8_e4m3 / __nv_fp8_e5m2 to float yields (cuda/src/ops/matmul.cu:161,170). */
EXPORT float oracle_e4m3_decode(uint8_t b) {
    int s = b >> 7, e = (b >> 3) & 0xf, m = b & 7;
    float v;
    if (e == 0xf && m == 7) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.f + m / 8.f, e - 7);
    return s ? -v : v;
}
EXPORT float oracle_e5m2_decode(uint8_t b) {
    int s = b >> 7, e = (b >> 2) & 0x1f, m = b & 3;
    float v;
    if (e == 0x1f) v = m ? NAN : INFINITY;
    else if (e == 0) v = ldexpf((float)m, -16);
    else v = ldexpf(1.f + m / 4.f, e - 15);
    return s ? -v : v;
}

/* fp8 e4m3fn encode, round-to-nearest-even, saturating to +-448 (the behaviour of constructing
 * __nv_fp8_e4m3 from float, used by the reference's aclnnCast: cuda/src/ops/cast.cu:79). */
EXPORT uint8_t oracle_e4m3_encode(float x) {
    uint32_t xb; memcpy(&xb, &x, 4);
    uint8_t s = (uint8_t)((xb >> 31) << 7);
    if ((xb & 0x7fffffffu) > 0x7f800000u) return (uint8_t)(s | 0x7f);
    float ax = fabsf(x);
    if (ax >= 464.f) return (uint8_t)(s | 0x7e);       /* above the 448/480 midpoint: saturate */
    if (ax < ldexpf(1.f, -10)) return s;                /* below half the smallest subnormal */
    int e; float fr = frexpf(ax, &e);                   /* ax = fr * 2^e, fr in [0.5,1) */
    int ue = e - 1;                                     /* unbiased exponent of 1.xxx form */
    float q;
    if (ue < -6) {                                      /* subnormal: multiples of 2^-9 */
        q = nearbyintf(ldexpf(ax, 9));
        if (q >= 8.f) return (uint8_t)(s | 0x08);
        return (uint8_t)(s | (uint8_t)q);
    }
    q = nearbyintf(ldexpf(fr, 4));                      /* 1.mmm * 8 in [8,16] */
    if (q >= 16.f) { q = 8.f; ue += 1; }
    if (ue > 8) return (uint8_t)(s | 0x7e);
    uint8_t code = (uint8_t)(((ue + 7) << 3) | ((int)q - 8));
    if (code > 0x7e) code = 0x7e;
    return (uint8_t)(s | code);
}

/* e8m0 block scale: 2^(e-127) (cuda/src/ops/matmul.cu:159,168; metal conv.mm e8m0()). */
static inline double e8m0(uint8_t e) { return ldexp(1.0, (int)e - 127); }

/* element decoders selected by an operand-kind code shared with the tests */
enum { MXK_E4M3 = 0, MXK_E5M2 = 1, MXK_E2M1 = 2 };
static inline double mx_elem(const uint8_t *p, int kind, int64_t idx) {
    if (kind == MXK_E2M1) {
        uint8_t byte = p[idx >> 1];
        return oracle_e2m1_decode((idx & 1) ? (byte >> 4) : (byte & 0xf));   /* element 0 = low nibble, subfp.cuh:10 */
    }
    return kind == MXK_E4M3 ? oracle_e4m3_decode(p[idx]) : oracle_e5m2_decode(p[idx]);
}

/* ---------------------------------------------------------------- operators */

/* Weight-only quantized matmul, W8A16 / W4A16.
 * Reference: metal/src/ops/conv.mm K_WQMM (lines 649-668) and cuda/src/ops/matmul.cu:331-352,
 * 733-747: wf = (w - offset[n]) * scale[n];  out = x @ wf.
 * Generalised the obvious way where the reference has no implementation: scale/offset may be
 * [G,N] with G = K/group (group-wise), and an optional bias[n] is added at the end.
 * x, scale, offset, bias arrive decoded to float (decoding fp16/bf16 to float is exact). */
EXPORT void oracle_wqbmm(const float *x, const uint8_t *w, int is_int4, const float *scale, const float *offset,
                         const float *bias, int64_t M, int64_t K, int64_t N, int64_t group, double *out) {
    if (group <= 0) group = K;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0;
            for (int64_t k = 0; k < K; ++k) {
                int64_t g = k / group;
                int wv = is_int4 ? int4_at(w, k * N + n) : (int)(int8_t)w[k * N + n];
                double of = offset ? (double)offset[g * N + n] : 0.0;
                double wf = ((double)wv - of) * (double)scale[g * N + n];
                acc += (double)x[m * K + k] * wf;
            }
            out[m * N + n] = acc + (bias ? (double)bias[n] : 0.0);
        }
}

/* W8A8 exact accumulation.  Reference: metal/src/ops/conv.mm K_QMM (612-623), long long sum;
 * cuda/src/ops/matmul.cu:825-842 computes the same int32 values with an int8 GEMM. */
EXPORT void oracle_qmm_acc(const int8_t *x, const int8_t *w, int64_t M, int64_t K, int64_t N, int32_t *acc) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            long long a = 0;
            for (int64_t k = 0; k < K; ++k) a += (long long)x[m * K + k] * (long long)w[k * N + n];
            acc[m * N + n] = (int32_t)a;
        }
}

/* W8A8 epilogue in fp32, exactly as the device does it so the final output can be compared
 * bit-for-bit: out = float(acc + bias[n]) * scale[n] * pertoken[m].
 * Reference: k_scale_i32, cuda/src/ops/matmul.cu:327-330 (float(c32) * float(scale[n])); bias and
 * per-token scale extend it in the order CANN documents (bias before the scales). */
EXPORT void oracle_qmm_epilogue(const int32_t *acc, const float *scale, const float *pertoken, const int32_t *bias,
                                int64_t M, int64_t N, float *out) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            int32_t a = acc[m * N + n] + (bias ? bias[n] : 0);
            float v = (float)a * scale[n];
            if (pertoken) v = v * pertoken[m];
            out[m * N + n] = v;
        }
}

/* MX block-scaled matmul.  Reference: metal/src/ops/conv.mm K_MXFP (712-732) and the CUDA dequant
 * kernels cuda/src/ops/matmul.cu:153-189: element * 2^(scale-127), one scale per 32 elements along
 * K; selfScale [M,K/32], otherScale [K/32,N]. */
EXPORT void oracle_mx_matmul(const uint8_t *a, int a_kind, const uint8_t *sa, const uint8_t *b, int b_kind,
                             const uint8_t *sb, int64_t M, int64_t K, int64_t N, double *out) {
    const int BLK = 32; int64_t nbk = K / BLK;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0;
            for (int64_t blk = 0; blk < nbk; ++blk) {
                double scA = e8m0(sa[m * nbk + blk]), scB = e8m0(sb[blk * N + n]);
                for (int t = 0; t < BLK; ++t) {
                    int64_t k = blk * BLK + t;
                    acc += mx_elem(a, a_kind, m * K + k) * scA * mx_elem(b, b_kind, k * N + n) * scB;
                }
            }
            out[m * N + n] = acc;
        }
}

/* int4 pack: out[i] = (in[2i+1] << 4) | (in[2i] & 0xF)  (cuda/src/ops/conv.cu:588-591). */
EXPORT void oracle_int4_pack(const int8_t *in, int64_t n_out, uint8_t *out) {
    for (int64_t i = 0; i < n_out; ++i) out[i] = (uint8_t)(((in[2 * i + 1] & 0xF) << 4) | (in[2 * i] & 0xF));
}

/* Position of logical block scale (row r, block b) in the 128x4 super-tile layout the reference
 * builds for hardware MX GEMMs (k_swizzle_scale, cuda/src/ops/matmul.cu:75-84). */
EXPORT int64_t oracle_scale_swizzle_index(int64_t r, int64_t b, int64_t nb) {
    int64_t nb_pad = (nb + 3) / 4 * 4, tiles_per_row = nb_pad / 4;
    int64_t tile = (r / 128) * tiles_per_row + (b / 4);
    int64_t rr = r % 128, c = b % 4;
    return tile * 512 + (rr % 32) * 16 + (rr / 32) * 4 + c;
}
