// Launch interface between the operator layer (ops_api.cu) and the kernel files.
// Plain pointers and sizes only; every launcher enqueues on the given stream and returns the
// launch status without synchronising.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace qmm {

// Element encodings understood by the kernels.
enum ElemType : int {
    ET_F32 = 0, ET_F16, ET_BF16, ET_I8, ET_I4, ET_I32, ET_E4M3, ET_E5M2, ET_E2M1, ET_E8M0, ET_U8, ET_NONE = -1
};

__host__ __device__ inline int elem_bits(int t) {
    switch (t) {
        case ET_F32: case ET_I32: return 32;
        case ET_F16: case ET_BF16: return 16;
        case ET_I4: case ET_E2M1: return 4;
        default: return 8;
    }
}

enum Epilogue : int {
    EPI_PLAIN = 0,   // out = acc (+ bias[n])                          (weight-only and MX matmuls)
    EPI_DEQ_I32,     // out = float(acc + bias_i32[n]) * scale[n] (* pertoken[m])   (W8A8)
    EPI_RAW_I32,     // out = acc (int32)                              (W8A8 accumulator dump)
};

// One matmul problem: out[b][M,N] = A[b][M,K] (x) B[b][K,N] with the dequantisation rules of the
// operator family selected by the element types.
struct MatmulArgs {
    const void *a = nullptr;       // [M,K] row-major
    const void *b = nullptr;       // [K,N] row-major (or [N,K] when b_transposed)
    void *out = nullptr;           // [M,N] row-major
    int a_type = ET_NONE, b_type = ET_NONE, out_type = ET_NONE;
    // weight-only: scale/offset [G,N] of sc_type, G = K/group.  W8A8: scale [N] of sc_type.
    const void *scale = nullptr;
    const void *offset = nullptr;
    int sc_type = ET_NONE;
    // MX: a_scale [M,K/32], b_scale [K/32,N], e8m0 bytes.
    const uint8_t *a_scale = nullptr;
    const uint8_t *b_scale = nullptr;
    const void *bias = nullptr;    // [N]; bias_type ET_I32 for W8A8, activation type otherwise
    int bias_type = ET_NONE;
    const float *pertoken = nullptr;  // [M] fp32 (W8A8)
    int epilogue = EPI_PLAIN;
    int64_t batch = 1, M = 0, N = 0, K = 0, group = 0;
    int64_t a_batch_stride = 0, b_batch_stride = 0, out_batch_stride = 0;  // elements
    bool b_transposed = false;
    bool b_nz = false;             // the weight is in its on-device format: int4 tile-packed (wq_mma.cu), or fp4 widened to e4m3 bytes (mx_tc.cu)
    bool accumulate = false;       // out = T(float(out) + float(T(result)))
    int split_k = 1;
    void *workspace = nullptr;
    uint64_t workspace_bytes = 0;
};

// Generic CUDA-core tile kernel: any shape, any supported type mix.  No workspace.
cudaError_t launch_generic(const MatmulArgs &p, cudaStream_t s);

// Streaming decode kernel for weight-only matmul at M <= gemv_max_m(): split-K over the grid,
// fp32 partials in `workspace`, reduced by a second kernel that applies bias and the output cast.
int gemv_max_m();
bool gemv_supported(const MatmulArgs &p);
int gemv_pick_split_k(const MatmulArgs &p);
uint64_t gemv_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_gemv(const MatmulArgs &p, cudaStream_t s);

// The same kernel with its split-K partial sums in a fixed array inside the library instead of a
// caller workspace (no allocation anywhere).  *too_large is set when the partial sums would not fit.
size_t noalloc_scratch_bytes();
cudaError_t launch_gemv_noalloc(MatmulArgs p, cudaStream_t s, bool *too_large);

// tcgen05 tensor-core kernel family.
bool tc_supported(const MatmulArgs &p);
void tc_plan(MatmulArgs &p);                 // fills split_k
uint64_t tc_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_tc(const MatmulArgs &p, cudaStream_t s);
// Dense tcgen05 kernel (tc.cu): W8A8, or 16-bit operands of one type.
bool dense_tc_supported(const MatmulArgs &p);
uint64_t dense_tc_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_dense_tc(const MatmulArgs &p, cudaStream_t s);
// Expand-then-dense path (dequant.cu): MX matmuls and large-M weight-only matmuls.
bool expand_supported(const MatmulArgs &p);
uint64_t expand_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_expand(const MatmulArgs &p, cudaStream_t s);
// Native block-scaled MX matmul (mx_tc.cu): tcgen05.mma kind::mxf8f6f4.block_scale with the e8m0 scales in tensor memory.
bool mx_native_supported(const MatmulArgs &p);
uint64_t mx_native_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_mx_native(const MatmulArgs &p, cudaStream_t s);
cudaError_t launch_mx_widen_fp4(const void *src, void *dst, int64_t elems, cudaStream_t s);
unsigned int mx_tc_device_status();
void mx_tc_device_status_reset();
// Persistent stream-K tensor-core kernel for weight-only matmuls (wq_tc.cu).
bool wq_tc_supported(const MatmulArgs &p);
uint64_t wq_tc_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_wq_tc(const MatmulArgs &p, cudaStream_t s);
unsigned int wq_tc_device_status();
void wq_tc_device_status_reset();
// Decode kernel for int4 weights at M <= 16 (wq_mma.cu): register dequant + mma.sync, stream-K.
bool wq_mma_supported(const MatmulArgs &p);
uint64_t wq_mma_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_wq_mma(const MatmulArgs &p, cudaStream_t s);
unsigned int wq_mma_device_status();
void wq_mma_device_status_reset();
// The tile-packed int4 weight layout the decode kernel streams with contiguous 16 KB copies: bytes it
// occupies for a [K,N] weight, the one-time re-layout from the caller's layout, and the way back.
uint64_t wq_nz_bytes(int64_t K, int64_t N);
cudaError_t launch_wq_pack_nz(const void *w_nd, void *w_nz, int64_t K, int64_t N, cudaStream_t s);
cudaError_t launch_wq_unpack_nz(const void *w_nz, void *w_nd, int64_t K, int64_t N, cudaStream_t s);
// Decode kernel for 3 to 16 rows on weights in the caller's layout (wq_rows.cu): activations in their own type.
bool wq_rows_supported(const MatmulArgs &p);
uint64_t wq_rows_workspace_bytes(const MatmulArgs &p);
cudaError_t launch_wq_rows(const MatmulArgs &p, cudaStream_t s);
unsigned int wq_rows_device_status();
void wq_rows_device_status_reset();
// Activation quantisers (dynquant.cu): the staged SwiGLU quantiser waits on its row copies with a limit.
unsigned int dynquant_device_status();
void dynquant_device_status_reset();
// 0, or the code of the first bounded wait that gave up on the current device (synchronises).
unsigned int tc_device_status();
// Clears the status words of every kernel family on the current device (synchronises).
void tc_device_status_reset();
// Gathering epilogue of the decode kernel: the calling thread's next decode launches also store their output rows into the
// peers' receive windows (see MmParams in wq_mma.cu).  nullptr clears.  consumed(): the thread's last launch did so.
struct DecodeGather {
    void *peer[8];
    const unsigned long long *calls;
    uint32_t nranks, rank;
    uint64_t buf_bytes;
    uint32_t f32, reserved;   // f32: packets carry one fp32 partial result each, also into the own window (all-reduce form)
};
void wq_mma_set_gather(const DecodeGather *g);
bool wq_mma_gather_consumed();
// bf16 activations [M,K] -> fp16 with a power-of-two scale per row (xh = x / rowscale exactly; dequant.cu).
cudaError_t launch_rows_bf16_to_scaled_f16(const void *x, void *xh, float *rowscale, int64_t M, int64_t K, cudaStream_t s);
void tc_reserve_sms(int n);   // the calling thread's dense-kernel plans leave n SMs free (0 = none)

// Host-side tally of kernels this library has launched (diagnostics for benchmarks).
void count_launch(int n = 1);
uint64_t launch_count();

// Small element-wise helpers.
cudaError_t launch_int4_pack(const int8_t *in, uint8_t *out, int64_t n_out, cudaStream_t s);
cudaError_t launch_fill_i64(int64_t *out, int64_t value, cudaStream_t s);
// residual add + RMS norm over rows of D elements (x, residual, outputs of one 16/32-bit float type).
cudaError_t launch_add_rmsnorm(const void *x, const void *res, const void *gamma, int type, int gamma_type, void *ysum, void *y,
                               int64_t rows, int64_t D, float eps, cudaStream_t s);
cudaError_t launch_qparam(const float *scale, const float *offset, int64_t *out, int64_t n, cudaStream_t s);
// Per-token dynamic int8 quantiser (dynquant.cu).
cudaError_t launch_dynamic_quant(const void *x, int x_type, int8_t *q, float *scale_out, int64_t rows, int64_t D, cudaStream_t s);
// SwiGLU + per-token int8: x [rows][2 D] -> q [rows][D], scale_out [rows].
cudaError_t launch_swiglu_quant(const void *x, int x_type, const float *dq, int8_t *q, float *scale_out, int64_t rows, int64_t D,
                                cudaStream_t s);
cudaError_t launch_dynamic_mx_quant(const void *x, int x_type, int8_t *q, float *scale_out, int64_t nblocks, int64_t blk, cudaStream_t s);
cudaError_t launch_cast(const void *in, int in_type, void *out, int out_type, int64_t n, cudaStream_t s);

}  // namespace qmm
