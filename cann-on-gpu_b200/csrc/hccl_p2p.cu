// Receive windows over peer memory (NVLink / NVSwitch) for the gathering epilogue of the decode matmul
// (aclnnB200WeightQuantMatmulAllGather): the [M, N/g] output shards of a column-partitioned layer are a few tens of
// kilobytes per call, where a library all-gather costs about 10 us by itself and 13-15 us behind a matmul.
//
// Every rank owns a "window": one cudaMalloc'd block with two receive buffers (used alternately) and a counter of
// completed calls.  The windows' IPC handles are exchanged once per communicator (through an NCCL all-gather), so every
// rank can store into every other rank's window.  The matmul kernel itself stores each finished output row into every
// peer's window as 8-byte packets {two 16-bit outputs, the call's number} with plain peer stores (no multicast, no
// fence: a packet is one store, so its number arrives with its data).  ll_unpack_kernel, enqueued behind the matmul
// with programmatic stream serialisation (its launch overlaps the matmul's tail), polls the packets of the other
// ranks in the local window until they carry this call's number (bounded), writes their payload into the caller's
// gathered tensor and advances the counter.  Nothing is allocated or synchronised per call, and the pair can be
// captured into a graph and replayed: the call number lives in device memory.
//
// Why two receive buffers are enough: a rank can be at most one call ahead of a peer (its unpack of call n + 1 ends only
// after every peer's packets of call n + 1 have arrived, which the peer sends from its matmul n + 1, i.e. after its own
// unpack of call n), so what a rank overwrites at call n + 2 was last read during call n.
//
// A plain (fence + flag) all-gather kernel over the same windows was measured first and dropped: 9.5 / 12.6 / 24.8 us
// for 7 / 28 / 128 KB per rank on two B200s against NCCL's 9.4 / 10.8 / 11.5 us.
//
// Failure handling: a poll gives up after about a second, records a code in a status word the host can read
// (HcclB200P2pStatus) and the kernel returns; the gathered tensor is then incomplete.  If any rank cannot open a peer's
// window the whole communicator keeps using NCCL (the ranks agree on that with an all-reduce).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>

#include "hccl_p2p.h"

namespace {

constexpr int P2P_MAX_RANKS = 8;
constexpr size_t P2P_BUF_BYTES = 8u << 20;           // one receive buffer: packets of a whole gathered result
constexpr unsigned long long P2P_WAIT_NS = 1000000000ull;

struct WindowView {
    uint8_t *win[P2P_MAX_RANKS];     // every rank's window as this process sees it (own window included)
    int nranks, rank;
};
// layout of a window: [receive buffer 0][receive buffer 1][completed calls u64][CTAs done u32]
__host__ __device__ inline size_t win_calls_off() { return 2 * P2P_BUF_BYTES; }
__host__ __device__ inline size_t win_bytes() { return win_calls_off() + 16; }

__device__ unsigned int g_p2p_status;

__device__ __forceinline__ unsigned long long p2p_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// gathered: [nranks][M][N] 16-bit elements; packet i of a receive buffer holds elements 2 i, 2 i + 1 of it.
__global__ void __launch_bounds__(256) ll_unpack_kernel(const WindowView w, uint32_t *gathered, unsigned long long pairs_per_rank,
                                                        unsigned long long wait_ns) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the matmul before this kernel has completed (its workspace is free again)
    uint8_t *mine = w.win[w.rank];
    unsigned long long *calls = reinterpret_cast<unsigned long long *>(mine + win_calls_off());
    unsigned int *done = reinterpret_cast<unsigned int *>(calls + 1);
    const unsigned long long call = *calls + 1;          // advanced by the last CTA of this kernel
    const uint2 *buf = reinterpret_cast<const uint2 *>(mine + (size_t)(call & 1ull) * P2P_BUF_BYTES);
    const unsigned long long total = pairs_per_rank * (unsigned long long)w.nranks;
    const unsigned long long own_lo = pairs_per_rank * (unsigned long long)w.rank, own_hi = own_lo + pairs_per_rank;
    bool ok = true;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total && ok; i += (unsigned long long)gridDim.x * blockDim.x) {
        if (i >= own_lo && i < own_hi) continue;         // the local shard was written by the matmul itself
        uint2 v;
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(buf + i) : "memory");
        if (v.y != (uint32_t)call) {
            const unsigned long long t0 = p2p_now();
            while (true) {
                asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(buf + i) : "memory");
                if (v.y == (uint32_t)call) break;
                if (p2p_now() - t0 > wait_ns) {
                    atomicCAS(&g_p2p_status, 0u, 0x500u + (unsigned)(i / pairs_per_rank));
                    ok = false;
                    break;
                }
            }
        }
        if (ok) gathered[i] = v.x;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {      // the kernel's last CTA closes the call
            *done = 0u;
            *calls = call;
        }
    }
}

// The all-reduce form of the receiver (K split over the ranks): every rank's matmul has stored its partial [M][N] result,
// unrounded, as packets {fp32 value, call number} into slot [rank] of every rank's window, its own included.
// out[i] = the sum over the ranks in rank order (fp32), rounded once to the 16-bit output type.  A thread takes two
// neighbouring outputs and writes them as one 32-bit word.
template <bool BF16>
__global__ void __launch_bounds__(256) ll_reduce_kernel(const WindowView w, uint32_t *out, unsigned long long pairs, unsigned long long wait_ns) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint8_t *mine = w.win[w.rank];
    unsigned long long *calls = reinterpret_cast<unsigned long long *>(mine + win_calls_off());
    unsigned int *done = reinterpret_cast<unsigned int *>(calls + 1);
    const unsigned long long call = *calls + 1;
    const uint2 *buf = reinterpret_cast<const uint2 *>(mine + (size_t)(call & 1ull) * P2P_BUF_BYTES);
    bool ok = true;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs && ok; i += (unsigned long long)gridDim.x * blockDim.x) {
        float acc[2] = {0.f, 0.f};
        for (int r = 0; r < w.nranks && ok; ++r) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint2 *pk = buf + ((unsigned long long)r * pairs + i) * 2 + h;
                uint2 v;
                asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(pk) : "memory");
                if (v.y != (uint32_t)call) {
                    const unsigned long long t0 = p2p_now();
                    while (true) {
                        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(pk) : "memory");
                        if (v.y == (uint32_t)call) break;
                        if (p2p_now() - t0 > wait_ns) {
                            atomicCAS(&g_p2p_status, 0u, 0x500u + (unsigned)r);
                            ok = false;
                            break;
                        }
                    }
                }
                acc[h] += __uint_as_float(v.x);
            }
        }
        if (ok) {
            if constexpr (BF16) {
                const __nv_bfloat162 hh = __floats2bfloat162_rn(acc[0], acc[1]);
                out[i] = *reinterpret_cast<const uint32_t *>(&hh);
            } else {
                const __half2 hh = __floats2half2_rn(acc[0], acc[1]);
                out[i] = *reinterpret_cast<const uint32_t *>(&hh);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0u;
            *calls = call;
        }
    }
}

struct Window {
    WindowView view{};
    bool usable = false;
};
std::mutex g_mu;
std::map<void *, Window> g_windows;   // per communicator

// Collective over the communicator: allocate, exchange handles, open the peers' windows, agree on the outcome.
Window make_window(const P2pNccl &nccl, void *comm, cudaStream_t s) {
    Window w;
    int n = 0, r = 0;
    if (nccl.comm_count(comm, &n) != 0 || nccl.comm_rank(comm, &r) != 0 || n < 2 || n > P2P_MAX_RANKS) return w;
    w.view.nranks = n; w.view.rank = r;
    int ok = 1;
    uint8_t *mine = nullptr;
    cudaIpcMemHandle_t *handles_dev = nullptr;
    cudaIpcMemHandle_t handles[P2P_MAX_RANKS];
    if (cudaMalloc(&mine, win_bytes()) != cudaSuccess) { ok = 0; mine = nullptr; }
    if (ok && (cudaMemset(mine, 0, win_bytes()) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)) ok = 0;   // cleared before any peer can write
    if (cudaMalloc(&handles_dev, sizeof(cudaIpcMemHandle_t) * n) != cudaSuccess) { ok = 0; handles_dev = nullptr; }
    cudaIpcMemHandle_t h{};
    if (ok && cudaIpcGetMemHandle(&h, mine) != cudaSuccess) ok = 0;
    if (handles_dev) {
        cudaMemcpy(handles_dev + r, &h, sizeof(h), cudaMemcpyHostToDevice);
        // every rank takes part in the exchange whatever its own state, so that nobody is left waiting
        const int rc = nccl.all_gather_bytes(comm, handles_dev + r, handles_dev, sizeof(h), s);
        if (rc != 0 || cudaStreamSynchronize(s) != cudaSuccess) ok = 0;
        if (cudaMemcpy(handles, handles_dev, sizeof(h) * n, cudaMemcpyDeviceToHost) != cudaSuccess) ok = 0;
    }
    for (int p = 0; p < n; ++p) w.view.win[p] = nullptr;
    if (ok) {
        w.view.win[r] = mine;
        for (int p = 0; p < n && ok; ++p) {
            if (p == r) continue;
            void *ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, handles[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { ok = 0; cudaGetLastError(); }
            w.view.win[p] = static_cast<uint8_t *>(ptr);
        }
    }
    // agree: the peer path is used only if it works on every rank
    int *flag_dev = reinterpret_cast<int *>(handles_dev);
    if (flag_dev) {
        cudaMemcpy(flag_dev, &ok, sizeof(int), cudaMemcpyHostToDevice);
        if (nccl.all_reduce_min_int(comm, flag_dev, s) != 0 || cudaStreamSynchronize(s) != cudaSuccess) ok = 0;
        int all = 0;
        if (cudaMemcpy(&all, flag_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) all = 0;
        ok = ok && all;
        cudaFree(handles_dev);
    }
    if (!ok) {
        for (int p = 0; p < n; ++p)
            if (p != r && w.view.win[p]) cudaIpcCloseMemHandle(w.view.win[p]);
        if (mine) cudaFree(mine);
        if (getenv("B200_HCCL_DBG")) fprintf(stderr, "[b200-hccl] rank %d: peer windows unavailable, all-gathers stay on NCCL\n", r);
        return w;
    }
    w.usable = true;
    return w;
}

}  // namespace

namespace {
// The communicator's window, set up collectively at first use (allocates and synchronises the stream, so not inside a
// stream capture: warm the operator up once before capturing).  nullptr: the peer path is not available.
Window *window_of(const P2pNccl &nccl, void *comm, cudaStream_t s) {
    static const bool enabled = [] { const char *e = getenv("B200_HCCL_P2P_GATHER"); return !(e && atoi(e) == 0); }();
    if (!enabled) return nullptr;
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_windows.find(comm);
    if (it == g_windows.end()) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return nullptr;
        it = g_windows.emplace(comm, make_window(nccl, comm, s)).first;
    }
    return it->second.usable ? &it->second : nullptr;
}
}  // namespace

bool p2p_gather_target(const P2pNccl &nccl, void *comm, cudaStream_t s, P2pGatherTarget *t) {
    Window *w = window_of(nccl, comm, s);
    if (!w) return false;
    for (int p = 0; p < P2P_MAX_RANKS; ++p) t->peer[p] = p < w->view.nranks ? w->view.win[p] : nullptr;
    t->calls = reinterpret_cast<const unsigned long long *>(w->view.win[w->view.rank] + win_calls_off());
    t->nranks = (uint32_t)w->view.nranks; t->rank = (uint32_t)w->view.rank;
    t->buf_bytes = P2P_BUF_BYTES;
    return true;
}

int p2p_unpack(const P2pNccl &nccl, void *comm, void *gathered, uint64_t elems_per_rank, cudaStream_t s) {
    Window *w = window_of(nccl, comm, s);
    if (!w || (elems_per_rank & 1) || elems_per_rank * 4 * (uint64_t)w->view.nranks > P2P_BUF_BYTES ||
        (reinterpret_cast<uintptr_t>(gathered) & 3))
        return -1;
    const unsigned long long pairs = elems_per_rank / 2, total = pairs * (unsigned long long)w->view.nranks;
    const unsigned grid = (unsigned)((total + 1023) / 1024 < 1 ? 1 : ((total + 1023) / 1024 > 64 ? 64 : (total + 1023) / 1024));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, ll_unpack_kernel, w->view, static_cast<uint32_t *>(gathered), pairs, P2P_WAIT_NS);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -1;
}

void p2p_forget(void *comm) {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_windows.find(comm);
    if (it == g_windows.end()) return;
    Window &w = it->second;
    if (w.usable) {
        cudaDeviceSynchronize();
        for (int p = 0; p < w.view.nranks; ++p)
            if (p != w.view.rank && w.view.win[p]) cudaIpcCloseMemHandle(w.view.win[p]);
        cudaFree(w.view.win[w.view.rank]);
    }
    g_windows.erase(it);
}

int p2p_reduce(const P2pNccl &nccl, void *comm, void *out, uint64_t elems, bool bf16, cudaStream_t s) {
    Window *w = window_of(nccl, comm, s);
    if (!w || (elems & 1) || elems * 8 * (uint64_t)w->view.nranks > P2P_BUF_BYTES || (reinterpret_cast<uintptr_t>(out) & 3)) return -1;
    const unsigned long long pairs = elems / 2;
    const unsigned long long want = (pairs + 511) / 512;
    const unsigned grid = (unsigned)(want < 1 ? 1 : (want > 64 ? 64 : want));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = bf16 ? cudaLaunchKernelEx(&cfg, ll_reduce_kernel<true>, w->view, static_cast<uint32_t *>(out), pairs, P2P_WAIT_NS)
                               : cudaLaunchKernelEx(&cfg, ll_reduce_kernel<false>, w->view, static_cast<uint32_t *>(out), pairs, P2P_WAIT_NS);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Test of the receiver's bounded poll without a second GPU and without faulting anything: a window of two "ranks" inside
// this process whose peer never sends, so the poll for its packets is a wait for something that never comes; it gives up
// after wait_ns, the kernel returns and the code is in the status word (returned, and cleared again).
unsigned int p2p_test_poll_runs_out(unsigned long long wait_ns) {
    WindowView v{};
    uint8_t *mine = nullptr;
    uint32_t *gathered = nullptr;
    if (cudaMalloc(&mine, win_bytes()) != cudaSuccess) return 0xFFFFFFFFu;
    if (cudaMalloc(&gathered, 2 * 16 * sizeof(uint32_t)) != cudaSuccess) { cudaFree(mine); return 0xFFFFFFFFu; }
    cudaMemset(mine, 0, win_bytes());
    v.nranks = 2; v.rank = 0; v.win[0] = mine; v.win[1] = mine;
    ll_unpack_kernel<<<1, 256>>>(v, gathered, 16, wait_ns);
    unsigned int code = 0xFFFFFFFFu;
    if (cudaDeviceSynchronize() == cudaSuccess) {
        code = p2p_status();
        const unsigned int zero = 0;
        cudaMemcpyToSymbol(g_p2p_status, &zero, sizeof(zero));
    }
    cudaFree(mine);
    cudaFree(gathered);
    return code;
}

unsigned int p2p_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_p2p_status, sizeof(v)) != cudaSuccess) return 0xFFFFFFFFu;
    return v;
}
