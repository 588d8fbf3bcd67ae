"""Benchmark of the quantized-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-sweep]

Workload (config.workload): the largest single-GPU configuration of the benchmark set -- the
Llama-70B-shaped gate/up projection as a W4A16 group-wise weight-only matmul, x bf16 [M=1, K=8192] @
int4 [8192, 28672] with bf16 scales per 128 rows of K (117 MB of packed weights per call, decode
shape, HBM-bound).  The smaller W4A16 configuration (4096 x 4096, 8.4 MB) fits in L2 and its ideal
time of 1.3 us is below a kernel launch, so it cannot show a memory roofline; it is reported in the
sweep instead.  One step is `passes` passes of the operator over a ring of R distinct weight sets whose
total size exceeds twice the L2, so every call streams its weights from HBM, and long enough (about
75 calls) that the timed region of the default run lasts tens of milliseconds.  The metric is weight
GB/s: packed weight bytes of the whole layer streamed per second.

With N > 1 (launched by torch.distributed.run) the FIXED [8192, 28672] layer is cut into N equal column
blocks, rank r owning weight[:, r*28672/N : (r+1)*28672/N] with the matching scale columns (strong
scaling, no collective on the data path): `value` is still whole-layer weight bytes per second, so
value(N) / (N * value(1)) is the efficiency of the partition.  Three more measurements ride in the
line's `sharded` object: the same calls followed by HcclAllGather of the bf16 output shards through
lib/libhccl.so (communicator from HcclGetRootInfo / HcclCommInitRootInfo, NCCL over NVLink), the
prefill form of the same shard (M = 4096), and the weak-scaling figure (every rank a whole 28672-column
problem).

--impl reference times the CPU restatement of the reference's algorithm (oracle/) on the host cores
for the same operator, on a column slice of the weight.  Synthetic seeded inputs throughout.
"""
import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

M, K, N, GROUP = 1, 8192, 28672, 128
RING_BYTES = 352_000_000  # a ring of weight sets holds at least this much: > 2 x 126 MB of L2
WEIGHT_BYTES = K * N // 2
CALLS_PER_STEP = 108      # about this many calls per step (a whole number of passes over the ring): 20 steps are over 50 ms
# Algorithmic bytes of one call: packed weights + group scales + activations + output.
ALGO_BYTES = WEIGHT_BYTES + (K // GROUP) * N * 2 + M * K * 2 + M * N * 2
WORKLOAD = ("W4A16 group-128 weight-only matmul, Llama-70B gate/up shape: x bf16 [1,8192] @ int4 [8192,28672], "
            "bf16 group scales, no offset, no bias")
CPU_SLICE_N = 2048  # columns of the weight the CPU legs work on
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic.json")   # ncu DRAM bytes per launch, with the commit captured at


def ring_size(n_cols):
    return max(3, math.ceil(RING_BYTES / (K * n_cols // 2)))


def ncu_traffic():
    """DRAM bytes (read + write) of one launch of the dominant kernel on this workload, from the tracked
    record of the last ncu capture; None when there is no record for the kernel."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f)["w4a16_g128_m1_8192x28672"]
        return rec["dram_bytes_per_launch"], rec
    except Exception:
        return None, None


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_ring(workloads, dev, rank, world, ring, m=M):
    """`ring` weight sets resident on the device: for world > 1 the rank's own column block of each set
    (drawn directly as a [K, N/world] problem; the layer is the concatenation of the ranks' blocks),
    plus the shared activations (the same on every rank)."""
    ns = N // world
    sets = []
    for i in range(ring):
        d = workloads.w4a16(M=1, K=K, N=ns, group=GROUP, seed=1004 + 1000 * rank + i, with_offset=False, with_bias=False)
        d["M"] = m
        d["x"] = torch.randn((m, K), generator=torch.Generator().manual_seed(5000 + i)).to(torch.bfloat16)
        sets.append({k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items() if k != "w_vals"})
    return sets


class Runner:
    """Pre-built aclTensor handles for the ring so the timed loop is phase 1 + phase 2 only.  With a
    communicator every call is followed by HcclAllGather of the output shard on the same stream."""

    def __init__(self, pkg, sets, dev, passes=1, gather=None, packed=True, fused=False):
        self.pkg, self.dev, self.passes, self.gather, self.fused = pkg, dev, passes, gather, fused
        m, ns = sets[0]["M"], sets[0]["N"]
        self.out = torch.empty((m, ns), dtype=torch.bfloat16, device=dev)
        self.t_out = pkg.AclTensor(self.out)
        self.items = []
        for d in sets:
            if packed:   # the weights in the library's on-device format, re-laid once at load time (aclnnTransMatmulWeight)
                if "w_nz" not in d:
                    d["w_nz"] = pkg.pack_weight_nz(d["w"], K, ns)
                tw = pkg.AclTensor(d["w_nz"], pkg.ACL_INT4, (K, ns), fmt=pkg.ACL_FORMAT_FRACTAL_NZ, storage=(d["w_nz"].numel() * 2,))
            else:
                tw = pkg.AclTensor(d["w"], pkg.ACL_INT4, (K, ns))
            self.items.append((pkg.AclTensor(d["x"]), tw, pkg.AclTensor(d["scale"]), None, None, d))
        self.ws = pkg.Workspace()
        if gather is not None:
            self.hccl, self.comm, world = gather
            self.gathered = torch.empty((world, m, ns), dtype=torch.bfloat16, device=dev)
            self.t_gathered = pkg.AclTensor(self.gathered)
            self.hccl_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")

    def call(self, i, x_handle=None):
        tx, tw, ts, to, tb, _ = self.items[i]
        if self.gather is not None and self.fused:
            # the gather fused into the matmul's epilogue: peer stores from the decode kernel + a receiver kernel
            with self.pkg.use_library(self.hccl_path):
                self.pkg.call("aclnnB200WeightQuantMatmulAllGather", x_handle or tx, tw, ts, to, tb, ctypes.c_int64(GROUP), self.comm,
                              self.t_gathered, workspace=self.ws, device=self.dev)
            return
        self.pkg.call("aclnnWeightQuantBatchMatmulV2Ex", x_handle or tx, tw, ts, to, tb, ctypes.c_int64(GROUP), self.t_out,
                      workspace=self.ws, device=self.dev)
        if self.gather is not None:
            st = self.hccl.HcclAllGather(ctypes.c_void_p(self.out.data_ptr()), ctypes.c_void_p(self.gathered.data_ptr()),
                                         ctypes.c_uint64(self.out.numel()), ctypes.c_int(11),   # HCCL_DATA_TYPE_BFP16
                                         self.comm, ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream))
            if st != 0:
                raise RuntimeError(f"HcclAllGather -> {st}")

    def step(self):
        for _ in range(self.passes):
            for i in range(len(self.items)):
                self.call(i)

    @property
    def calls_per_step(self):
        return self.passes * len(self.items)

    def capture(self):
        """One step as a CUDA graph: phase 2 neither allocates nor synchronises, so the calls can be
        captured; replaying removes the host's per-call overhead from the timing.  Returns False (and
        keeps direct calls) if the capture is refused."""
        lib = self.pkg.load()
        n0 = lib.aclnnB200KernelLaunchCount()
        try:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                self.step()
            self.replay = self.graph.replay
            captured = True
        except Exception:
            torch.cuda.synchronize()
            self.graph, self.replay, captured = None, self.step, False
            n0 = lib.aclnnB200KernelLaunchCount()
            self.step()
        self.launches_per_step = lib.aclnnB200KernelLaunchCount() - n0
        return captured


def hccl_communicator(pkg, world, rank, dev):
    """A communicator of the library's own collective layer, set up the way an HCCL program does it
    (rank 0 takes HcclGetRootInfo, the blob travels out of band -- here a torch broadcast -- and every
    rank calls HcclCommInitRootInfo)."""
    import torch.distributed as dist
    hccl_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
    if not os.path.exists(hccl_path):
        raise RuntimeError(f"{hccl_path} is missing: run __graft_entry__.build()")
    hccl = pkg.load(hccl_path)
    info = ctypes.create_string_buffer(4108)
    if rank == 0 and hccl.HcclGetRootInfo(info) != 0:
        raise RuntimeError("HcclGetRootInfo failed")
    blob = torch.frombuffer(bytearray(info.raw), dtype=torch.uint8).to(dev)
    dist.broadcast(blob, src=0)
    info.raw = bytes(blob.cpu().numpy().tobytes())
    comm = ctypes.c_void_p()
    st = hccl.HcclCommInitRootInfo(ctypes.c_uint32(world), info, ctypes.c_uint32(rank), ctypes.byref(comm))
    if st != 0:
        raise RuntimeError(f"HcclCommInitRootInfo -> {st}")
    return hccl, comm


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    return rank, world, local


def max_over_ranks(ms, world, dev):
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def timed(fn, steps, world, dev):
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    barrier(world)
    return max_over_ranks(ms, world, dev)


REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libascendcl_ref.so")

# bound of a sweep row -> (key of the measured peak, multiplier, unit, note)
BOUNDS = {
    "hbm": ("hbm_gbs", 1.0, "GB/s", "measured copy bandwidth"),
    "tensor bf16": ("bf16_tflops", 1.0, "TFLOP/s", "measured bf16 burst"),
    "tensor int8": ("bf16_tflops", 2.0, "TOP/s", "2 x measured bf16 burst (proxy: no measured int8 peak)"),
    "tensor fp8": ("bf16_tflops", 2.0, "TFLOP/s", "2 x measured bf16 burst (proxy: no measured fp8 peak)"),
}


def time_graph(calls, reps, allow_eager=False):
    """Average microseconds per call of `calls` (zero-argument callables, one per weight set): one CUDA
    graph over the list, replayed `reps` times between CUDA events."""
    for c in calls:
        c()
    torch.cuda.synchronize()
    mode = "graph"
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for c in calls:
                c()
        run = g.replay
    except Exception:
        if not allow_eager:
            raise
        torch.cuda.synchronize()
        mode = "eager"

        def run():
            for c in calls:
                c()
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(calls)), mode


def sweep_cases(workloads):
    """The other benchmark configurations.  Each case: name, bound, flops, weight bytes, algorithmic bytes,
    reps, a maker of this library's calls, and a maker of the closest form the reference's own CUDA
    backend accepts (fp16 activations, per-channel [N] scales, fp16 output, same-kind MX operands:
    cuda/src/ops/matmul.cu:761-767,802-807,437,491 of the reference) or None."""
    cases = []

    def wq(name, bound, sets_fn, int4, group, m, k, n, reps, with_ref=True):
        wb = k * n // 2 if int4 else k * n
        scale_rows = (k // group) if group else 1

        def mine(pkg, dev):
            calls, ws = [], pkg.Workspace()
            for d in sets_fn():
                out = torch.empty((m, n), dtype=d["x"].dtype, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev), pkg.ACL_INT4 if int4 else pkg.ACL_INT8, (k, n)),
                        pkg.AclTensor(d["scale"].to(dev)), pkg.AclTensor(d["offset"].to(dev)) if d["offset"] is not None else None,
                        pkg.AclTensor(d["bias"].to(dev)) if d["bias"] is not None else None, ctypes.c_int64(group), pkg.AclTensor(out)]
                calls.append(lambda a=args: pkg.call("aclnnWeightQuantBatchMatmulV2Ex", *a, workspace=ws, device=dev))
            return calls

        def ref(pkg, dev):
            calls, ws = [], pkg.Workspace()
            for d in sets_fn()[:2]:
                sc = d["scale"].reshape(-1, n)[0].half().contiguous()
                of = d["offset"].reshape(-1, n)[0].half().contiguous() if d["offset"] is not None else None
                out = torch.empty((m, n), dtype=torch.float16, device=dev)
                args = [pkg.AclTensor(d["x"].half().to(dev)), pkg.AclTensor(d["w"].to(dev), pkg.ACL_INT4 if int4 else pkg.ACL_INT8, (k, n)),
                        pkg.AclTensor(sc.to(dev)), pkg.AclTensor(of.to(dev)) if of is not None else None, pkg.AclTensor(out)]
                calls.append(lambda a=args: pkg.call("aclnnWeightQuantBatchMatmul", *a, workspace=ws, device=dev))
            return calls

        es = 2
        abytes = wb + scale_rows * n * es * (2 if "+offset" in name else 1) + m * k * es + m * n * es
        cases.append(dict(name=name, bound=bound, flops=2 * m * k * n, wbytes=wb, abytes=abytes, reps=reps, mine=mine,
                          ref=ref if with_ref else None,
                          ref_form="fp16 activations and output, per-channel [N] scale" + (" and offset" if "+offset" in name else "")))

    def i8(name, bound, m, reps):
        k, n = 4096, 14336

        def mine(pkg, dev):
            calls, ws = [], pkg.Workspace()
            for i in range(5):
                d = workloads.w8a8(M=m, seed=1002 + i)
                out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev)), None,
                        pkg.AclTensor(d["pertoken"].to(dev)), pkg.AclTensor(d["bias"].to(dev)), pkg.AclTensor(out)]
                calls.append(lambda a=args: pkg.call("aclnnQuantMatmulV4Ex", *a, workspace=ws, device=dev))
            return calls

        def ref(pkg, dev):
            calls, ws = [], pkg.Workspace()
            for i in range(2):
                d = workloads.w8a8(M=m, seed=1002 + i, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
                out = torch.empty((m, n), dtype=torch.float16, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev)), pkg.AclTensor(out)]
                calls.append(lambda a=args: pkg.call("aclnnQuantMatmul", *a, workspace=ws, device=dev))
            return calls

        cases.append(dict(name=name, bound=bound, flops=2 * m * k * n, wbytes=k * n, abytes=k * n + m * k + m * n * 2 + n * 8 + m * 4,
                          reps=reps, mine=mine, ref=ref, ref_form="fp16 [N] scale, fp16 output, no per-token scale, no bias"))

    # config 0: W8A16 M=1 K=1024 N=3072 (3 MB per call: L2-resident and launch-bound)
    wq("cfg0 W8A16 per-channel M=1 K=1024 N=3072 fp16", "hbm", lambda: [workloads.w8a16(seed=1000 + i) for i in range(32)],
       False, 0, 1, 1024, 3072, 20)
    # config 1: W4A16 g128 K=4096 N=4096 with offset and bias, M = 1 / 16 / 128 (8.4 MB per call)
    for m in (1, 16, 128):
        wq(f"cfg1 W4A16 g128 M={m} K=4096 N=4096 bf16 +offset +bias", "hbm",
           lambda m=m: [workloads.w4a16(M=m, seed=1001 + i) for i in range(32)], True, 128, m, 4096, 4096, 10)
    # config 4: Llama-70B shapes, W4A16 g128, no offset
    for which, k, n in (("gate/up", 8192, 28672), ("down", 28672, 8192)):
        for m in (32, 512, 4096):
            if which == "down" and m == 4096:
                continue
            wq(f"cfg4 W4A16 g128 {which} M={m} K={k} N={n} bf16", "hbm" if m < 512 else "tensor bf16",
               lambda m=m, which=which: [workloads.llama70b_shard(m, "gate_up" if which == "gate/up" else "down", seed=1004 + i) for i in range(3)],
               True, 128, m, k, n, 5 if m < 4096 else 3)
    # config 2: W8A8 K=4096 N=14336, per-token x per-channel scales, int32 bias, bf16 out
    for m in (1, 8, 256, 2048, 4096):
        i8(f"cfg2 W8A8 M={m} K=4096 N=14336 bf16 out", "hbm" if m <= 256 else "tensor int8", m, 5)
    return cases


def quantiser_rows(pkg, dev):
    """The activation quantisers in front of config 2 (HBM-bound; bytes are everything moved)."""
    rows = []
    for m in (2048, 4096):
        calls, ws = [], pkg.Workspace()
        for i in range(12):   # 12 x (32 MB in + 16 MB out) > 2 x L2
            x = torch.randn((m, 4096), generator=torch.Generator().manual_seed(3000 + i)).to(torch.bfloat16).to(dev)
            q = torch.empty((m, 4096), dtype=torch.int8, device=dev)
            sc = torch.empty((m,), dtype=torch.float32, device=dev)
            args = [pkg.AclTensor(x), pkg.AclTensor(q), pkg.AclTensor(sc)]
            calls.append(lambda a=args: pkg.call("aclnnDynamicQuant", *a, workspace=ws, device=dev))
        rows.append((f"DynamicQuant per-token bf16 [{m},4096] -> int8 (feeds cfg2)", calls, m * 4096 * 3 + m * 4, 10))
    m = 2048
    calls, ws = [], pkg.Workspace()
    for i in range(3):   # 3 x (117 MB in + 29 MB out) > 2 x L2
        x = torch.randn((m, 28672), generator=torch.Generator().manual_seed(3100 + i)).to(torch.bfloat16).to(dev)
        q = torch.empty((m, 14336), dtype=torch.int8, device=dev)
        sc = torch.empty((m,), dtype=torch.float32, device=dev)
        args = [pkg.AclTensor(x), pkg.AclTensor(q), pkg.AclTensor(sc)]
        calls.append(lambda a=args: pkg.call("aclnnSwiGluQuant", *a, workspace=ws, device=dev))
    rows.append((f"SwiGluQuant bf16 [{m},28672] -> int8 [{m},14336]", calls, m * 14336 * 5 + m * 4, 10))
    return rows


def mx_case(workloads, a_fp4, b_fp4, entry, out_dtype, widen_b=False):
    """widen_b: the fp4 weight in its on-device format (aclnnTransMatmulWeight once, outside the timed region)."""
    def make(pkg, dev):
        ws = pkg.Workspace()
        d = workloads.mx(a_fp4=a_fp4, b_fp4=b_fp4)
        ak = pkg.ACL_FLOAT4_E2M1 if a_fp4 else pkg.ACL_FLOAT8_E4M3FN
        bk = pkg.ACL_FLOAT4_E2M1 if b_fp4 else pkg.ACL_FLOAT8_E4M3FN
        out = torch.empty((4096, 8192), dtype=out_dtype, device=dev)
        b = d["b"].reshape(-1).to(dev)
        if widen_b:
            b = pkg.widen_fp4_weight(b, 8192, 8192)
            tb = pkg.AclTensor(b, bk, (8192, 8192), fmt=pkg.ACL_FORMAT_FRACTAL_NZ, storage=(b.numel() * 2,))
        else:
            tb = pkg.AclTensor(b, bk, (8192, 8192))
        args = [pkg.AclTensor(d["a"].reshape(-1).to(dev), ak, (4096, 8192)), pkg.AclTensor(d["sa"].to(dev), pkg.ACL_FLOAT8_E8M0, (4096, 256)),
                tb, pkg.AclTensor(d["sb"].to(dev), pkg.ACL_FLOAT8_E8M0, (256, 8192)),
                pkg.AclTensor(out)]
        return [lambda a_=args: pkg.call(entry, *a_, workspace=ws, device=dev)]
    return make


def ref_cuda_worker(only):
    """Child process: times the reference's own CUDA backend (oracle/_ref, built from the reference's
    sources by oracle/build_ref.sh) on the closest form of each sweep case it accepts, one JSON line per
    case.  A process of its own so that nothing the reference's code does can lose the parent's line."""
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    pkg = ge.load_package()
    from cann_on_gpu_b200 import workloads
    todo = [(c["name"], c["ref"], c["ref_form"]) for c in sweep_cases(workloads) if c["ref"] is not None]
    todo.append(("cfg3 MXFP8xMXFP4 M=4096 K=8192 N=8192 bf16 out", mx_case(workloads, False, False, "aclnnMatmulMxFp8Hw", torch.float16),
                 "MXFP8 x MXFP8 (the reference takes no mixed operands), fp16 output, Hw entry: per-call transpose + scale re-layout + cuBLASLt block-scaled GEMM"))
    for name, make, form in todo:
        if only is not None and only not in name:
            continue
        row = {"case": name, "form": form}
        try:
            with pkg.use_library(REF_LIB):
                us, mode = time_graph(make(pkg, dev), 2, allow_eager=True)
            row.update(us=round(us, 2), launch=mode)
        except Exception as e:
            row["error"] = repr(e)[:200]
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        print("REFROW " + json.dumps(row), flush=True)


def ref_cuda_times(only=None):
    """{case name: row} from the child process, or a one-line reason why there are none."""
    if not os.path.exists(REF_LIB):
        return "unavailable: oracle/_ref/libascendcl_ref.so not built (needs the reference's source tree at build time)"
    cmd = [sys.executable, os.path.abspath(__file__), "--ref-cuda-worker"] + (["--sweep-only", only] if only else [])
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=600)
    except Exception as e:
        return "unavailable: " + repr(e)[:120]
    rows = {}
    for ln in r.stdout.splitlines():
        if ln.startswith("REFROW "):
            d = json.loads(ln[7:])
            rows[d.pop("case")] = d
    return rows if rows else f"unavailable: worker exit code {r.returncode}"


def sweep(pkg, workloads, dev, pk, only=None, with_ref=True):
    """Every other configuration, each captured as one CUDA graph over a ring of distinct weight sets
    (larger than L2 where memory allows) and timed with CUDA events.  Every row names its bound, the
    peak it is held against and the fraction reached; `ref_cuda` is the reference's own CUDA backend on
    the closest form it accepts, on the same GPU."""
    rows = []

    def add(name, us, flops, wbytes, abytes, bound, ring):
        key, mult, unit, note = BOUNDS[bound]
        peak = pk[key] * mult
        achieved = abytes / us / 1e3 if bound == "hbm" else flops / us / 1e6
        rows.append({"case": name, "us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "weight_gbs": round(wbytes / us / 1e3, 1),
                     "ring": ring, "bound": bound, "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": unit,
                     "frac": round(achieved / peak, 3), "peak_is": note})

    if only is not None and only.startswith("case:"):
        # one custom case, e.g. --sweep-only case:w4,128,8192,28672,128  (kind w4 | w8 | i8, M, K, N[, group])
        kind, m, k, n, *rest = only[5:].split(",")
        m, k, n = int(m), int(k), int(n)
        group = int(rest[0]) if rest else 128
        wb = k * n // 2 if kind == "w4" else k * n
        ring = max(2, min(32, 300_000_000 // wb + 1))
        ws = pkg.Workspace()
        calls = []
        for i in range(ring):
            if kind in ("w4", "w8"):
                d = (workloads.w4a16(M=m, K=k, N=n, seed=1100 + i, group=group, with_offset=False, with_bias=False) if kind == "w4"
                     else workloads.w8a16(M=m, K=k, N=n, seed=1100 + i, dtype=torch.bfloat16))
                out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev), pkg.ACL_INT4 if kind == "w4" else pkg.ACL_INT8, (k, n)),
                        pkg.AclTensor(d["scale"].to(dev)), None, None, ctypes.c_int64(d["group"]), pkg.AclTensor(out)]
                calls.append(lambda a=args: pkg.call("aclnnWeightQuantBatchMatmulV2Ex", *a, workspace=ws, device=dev))
            else:
                d = workloads.w8a8(M=m, K=k, N=n, seed=1100 + i)
                out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev)), None,
                        pkg.AclTensor(d["pertoken"].to(dev)), pkg.AclTensor(d["bias"].to(dev)), pkg.AclTensor(out)]
                calls.append(lambda a=args: pkg.call("aclnnQuantMatmulV4Ex", *a, workspace=ws, device=dev))
        us, _ = time_graph(calls, 5)
        add(f"{kind} M={m} K={k} N={n} group={group} bf16", us, 2 * m * k * n, wb, wb + m * k * 2 + m * n * 2,
            "hbm" if m < 512 else ("tensor int8" if kind == "i8" else "tensor bf16"), ring)
        return rows

    def wanted(name):
        return only is None or only in name

    try:
        for c in sweep_cases(workloads):
            if not wanted(c["name"]):
                continue
            calls = c["mine"](pkg, dev)
            us, _ = time_graph(calls, c["reps"])
            add(c["name"], us, c["flops"], c["wbytes"], c["abytes"], c["bound"], len(calls))
            del calls
            torch.cuda.empty_cache()
        for name, calls, nbytes, reps in (quantiser_rows(pkg, dev) if only is None or "Quant" in (only or "") else []):
            if not wanted(name):
                continue
            us, _ = time_graph(calls, reps)
            add(name, us, 0, nbytes, nbytes, "hbm", len(calls))
        torch.cuda.empty_cache()
        name = "cfg3 MXFP8xMXFP4 M=4096 K=8192 N=8192 bf16 out"
        if wanted(name):
            us, _ = time_graph(mx_case(workloads, False, True, "aclnnMatmulMxFp8", torch.bfloat16, widen_b=True)(pkg, dev), 3)
            add(name, us, 2 * 4096 * 8192 * 8192, 8192 * 8192 // 2, 4096 * 8192 + 8192 * 8192 // 2 + 4096 * 8192 * 2, "tensor fp8", 1)
            rows[-1]["weight_format"] = "fp4 weight widened once at load time by aclnnTransMatmulWeight (ACL_FORMAT_FRACTAL_NZ)"
            torch.cuda.empty_cache()
            us2, _ = time_graph(mx_case(workloads, False, True, "aclnnMatmulMxFp8", torch.bfloat16)(pkg, dev), 3)
            rows[-1]["us_with_per_call_widening"] = round(us2, 2)
    except Exception as e:  # a sweep failure must not lose the headline line
        rows.append({"error": repr(e)[:300]})
    if with_ref:
        torch.cuda.empty_cache()
        ref = ref_cuda_times(only)
        for r in rows:
            if "case" not in r:
                continue
            if isinstance(ref, str):
                r["ref_cuda"] = ref
            elif r["case"] in ref:
                r["ref_cuda"] = ref[r["case"]]
    return rows


def _cpu_problem():
    """The CPU legs work on a column slice of one weight set of the device arm's ring."""
    ge.load_package()
    from cann_on_gpu_b200 import workloads
    d = workloads.w4a16(M=M, K=K, N=CPU_SLICE_N, group=GROUP, seed=1004, with_offset=False, with_bias=False)
    return (d["x"].float().numpy(), d["w"].numpy(), True, d["scale"].float().numpy(), None, None, M, K, CPU_SLICE_N, GROUP)


def cpu_baseline(seconds=12.0):
    """The CPU restatement (BLAS-backed form) of the same operator on the host cores."""
    o = ge.load_oracle()
    torch.set_num_threads(os.cpu_count() or 1)
    args = _cpu_problem()
    o.wqbmm_torch(*args)
    n, t0 = 0, time.perf_counter()
    while True:
        o.wqbmm_torch(*args)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or n >= 200:
            break
    return {"value": round(n * K * CPU_SLICE_N // 2 / dt / 1e9, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n} passes of the PyTorch-CPU restatement (fp32 dequant + matmul, all cores) over a {K}x{CPU_SLICE_N} column slice of one weight set at M={M} "
                      f"({dt:.1f} s)"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    o = ge.load_oracle()
    torch.set_num_threads(os.cpu_count() or 1)   # torch.distributed.run pins OMP_NUM_THREADS to 1
    a = _cpu_problem()
    for _ in range(max(1, args.warmup)):
        o.wqbmm_torch(*a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.wqbmm_torch(*a)
    dt = time.perf_counter() - t0
    v = args.steps * (K * CPU_SLICE_N // 2) / dt / 1e9
    sample = (f"each step = one pass of the PyTorch-CPU restatement (fp32 dequant + matmul, all cores) over a {K}x{CPU_SLICE_N} column slice ({CPU_SLICE_N}/{N} of one of the "
              f"weight sets of the device arm's ring)")
    print(json.dumps({
        "impl": "reference", "metric": "w4a16_g128_weight_stream", "value": round(v, 4), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M, "K": K, "N": N, "group": GROUP},
        "cpu_baseline": {"value": round(v, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--ring", type=int, default=0, help="weight sets in the ring (default: enough for 2 x L2)")
    ap.add_argument("--passes", type=int, default=0, help="passes over the ring per step (default: about 108 calls per step)")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip the reference-CUDA-backend column of the sweep")
    ap.add_argument("--sweep-only", default=None, help="run only the sweep cases whose name contains this text, and nothing else; "
                         "case:<w4|w8|i8>,M,K,N[,group] times one custom shape instead")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ref-cuda-worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.ref_cuda_worker:
        ref_cuda_worker(args.sweep_only)
        return
    args.warmup = max(3, args.warmup)

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    pkg = ge.load_package()
    from cann_on_gpu_b200 import workloads
    lib = pkg.load()
    lib.aclnnB200KernelLaunchCount.restype = ctypes.c_uint64
    pk = peaks()

    if args.sweep_only is not None:
        print(json.dumps({"sweep": sweep(pkg, workloads, dev, pk, only=args.sweep_only, with_ref=not args.no_ref_cuda)}))
        return
    assert N % world == 0 and (N // world) % 256 == 0, "column blocks of whole 256-column tiles"
    ns = N // world
    ring = args.ring or ring_size(ns)
    passes = args.passes or max(1, round(CALLS_PER_STEP / ring))
    sets = make_ring(workloads, dev, rank, world, ring)
    runner = Runner(pkg, sets, dev, passes)
    for _ in range(args.warmup):
        runner.step()
    torch.cuda.synchronize()

    runner.capture()
    for _ in range(args.warmup):
        runner.replay()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # bring the clocks back up after the pause (an idle GPU drops them within milliseconds)
    t_spin = time.perf_counter()
    while time.perf_counter() - t_spin < 0.2:
        runner.replay()
    torch.cuda.synchronize()
    ms = timed(runner.replay, args.steps, world, dev)
    launches = runner.launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    calls = args.steps * runner.calls_per_step
    value = calls * WEIGHT_BYTES / ms / 1e6  # GB/s of the whole layer (all ranks' column blocks together)

    # the same calls on weights left in the caller's [K,N] layout (no pre-pack)
    nd_runner = Runner(pkg, sets, dev, passes, packed=False)
    for _ in range(args.warmup):
        nd_runner.step()
    torch.cuda.synchronize()
    nd_runner.capture()
    for _ in range(args.warmup):
        nd_runner.replay()
    ms_nd = timed(nd_runner.replay, args.steps, world, dev)
    del nd_runner

    # ---- the other measurements of the partition (every N, so that t_1 / (N t_N) can be formed per variant)
    sharded = {"columns_per_rank": ns, "m1_us_per_call": round(ms / calls * 1e3, 3)}
    if world > 1:
        try:
            gather = hccl_communicator(pkg, world, rank, dev) + (world,)
            g_runner = Runner(pkg, sets, dev, passes, gather=gather)
            for _ in range(args.warmup):
                g_runner.step()
            torch.cuda.synchronize()
            captured = g_runner.capture()
            for _ in range(args.warmup):
                g_runner.replay()
            ms_g = timed(g_runner.replay, args.steps, world, dev)
            sharded["m1_gathered_us_per_call"] = round(ms_g / calls * 1e3, 3)
            sharded["m1_gathered_value_gbs"] = round(calls * WEIGHT_BYTES / ms_g / 1e6, 2)
            sharded["gather"] = ("HcclAllGather of the bf16 output shards after every call, same stream, through lib/libhccl.so "
                                 "(NCCL); " + ("captured in the step's CUDA graph" if captured else "direct calls (capture refused)"))
            del g_runner
            # the same with the gather fused into the matmul (aclnnB200WeightQuantMatmulAllGather)
            f_runner = Runner(pkg, sets, dev, passes, gather=gather, fused=True)
            for _ in range(args.warmup):
                f_runner.step()
            torch.cuda.synchronize()
            f_runner.capture()
            for _ in range(args.warmup):
                f_runner.replay()
            ms_f = timed(f_runner.replay, args.steps, world, dev)
            gather[0].aclnnB200FusedGatherCount.restype = ctypes.c_uint64
            sharded["m1_fused_gather_us_per_call"] = round(ms_f / calls * 1e3, 3)
            sharded["m1_fused_gather_value_gbs"] = round(calls * WEIGHT_BYTES / ms_f / 1e6, 2)
            sharded["fused_gather"] = ("aclnnB200WeightQuantMatmulAllGather: the decode kernel stores its output rows into the peers' receive "
                                       "windows (peer memory, 8-byte packets), a receiver kernel behind it fills the gathered tensor; "
                                       f"{int(gather[0].aclnnB200FusedGatherCount())} calls took the fused form")
            del f_runner
        except Exception as e:
            sharded.setdefault("m1_gathered_us_per_call", None)
            sharded["gather"] = sharded.get("gather", "") + " failed: " + repr(e)[:200]
            gather = None if "m1_gathered_us_per_call" not in sharded or sharded["m1_gathered_us_per_call"] is None else gather
    else:
        gather = None
    # prefill form of the same shard: M = 4096 rows against two of the ring's weight sets
    try:
        xs = [torch.randn((4096, K), generator=torch.Generator().manual_seed(5100 + i)).to(torch.bfloat16).to(dev) for i in range(2)]
        p_sets = [dict(sets[i], M=4096, x=xs[i]) for i in range(2)]
        p_runner = Runner(pkg, p_sets, dev, 1)
        for _ in range(3):
            p_runner.step()
        torch.cuda.synchronize()
        p_runner.capture()
        for _ in range(3):
            p_runner.replay()
        p_steps = 5
        ms_p = timed(p_runner.replay, p_steps, world, dev)
        us_p = ms_p / (p_steps * 2) * 1e3
        sharded["m4096_us_per_call"] = round(us_p, 2)
        sharded["m4096_tflops"] = round(2 * 4096 * K * N / us_p / 1e6, 1)   # whole layer, all ranks
        if gather is not None:
            pg = Runner(pkg, p_sets, dev, 1, gather=gather)
            for _ in range(3):
                pg.step()
            torch.cuda.synchronize()
            pg.capture()
            for _ in range(3):
                pg.replay()
            ms_pg = timed(pg.replay, p_steps, world, dev)
            sharded["m4096_gathered_us_per_call"] = round(ms_pg / (p_steps * 2) * 1e3, 2)
            del pg
        del p_runner, p_sets, xs
    except Exception as e:
        sharded["m4096_us_per_call"] = None
        sharded["m4096_error"] = repr(e)[:200]
    torch.cuda.empty_cache()
    if world > 1:
        # weak scaling, for comparison: every rank a whole 28672-column problem (its own block repeated)
        try:
            w_sets = []
            for i in range(3):
                d = sets[i]
                w_sets.append(dict(d, N=N, w=d["w"].reshape(K, ns // 2).repeat(1, world).reshape(-1).contiguous(),
                                   scale=d["scale"].repeat(1, world).contiguous()))
            w_runner = WeakRunner(pkg, w_sets, dev, 8)
            for _ in range(3):
                w_runner.step()
            torch.cuda.synchronize()
            w_runner.capture()
            for _ in range(3):
                w_runner.replay()
            ms_w = timed(w_runner.replay, 5, world, dev)
            sharded["weak_value_gbs"] = round(world * 5 * w_runner.calls_per_step * WEIGHT_BYTES / ms_w / 1e6, 2)
            sharded["weak"] = "every rank streams a whole [8192, 28672] layer (no partition): aggregate weight GB/s"
            del w_runner, w_sets
        except Exception as e:
            sharded["weak_value_gbs"] = None
            sharded["weak_error"] = repr(e)[:200]
        torch.cuda.empty_cache()

    if world > 1 and gather is not None:
        # The reference's other multi-GPU form, for comparison: K split over the ranks and an all-reduce of the
        # output (W8A8 prefill 4096 x 4096 x 14336, bf16 out), as the plain sequence (the library's default) and with the
        # all-reduce of a row chunk overlapping the next chunk's matmul (two chunks, 20 SMs left to the all-reduce).
        try:
            hccl_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
            comm = gather[1]
            kr = 4096 // world
            gq = torch.Generator().manual_seed(5200 + rank)
            qx = torch.randint(-127, 128, (4096, kr), generator=gq, dtype=torch.int8).to(dev)
            qw = torch.randint(-127, 128, (kr, 14336), generator=gq, dtype=torch.int8).to(dev)
            qs = (torch.rand(14336, generator=torch.Generator().manual_seed(5199)) * 1e-3 + 1e-4).to(torch.bfloat16).to(dev)
            qo = torch.empty((4096, 14336), dtype=torch.bfloat16, device=dev)
            ws_q = pkg.Workspace()
            targs = [pkg.AclTensor(qx), pkg.AclTensor(qw), pkg.AclTensor(qs), comm, pkg.AclTensor(qo)]

            def ksplit_step():
                with pkg.use_library(hccl_path):
                    for _ in range(4):
                        pkg.call("aclnnQuantMatmulAllReduce", *targs, workspace=ws_q, device=dev)
            res = {}
            for label, chunks in (("plain", None), ("overlapped", "2")):
                if chunks is None:
                    os.environ.pop("B200_HCCL_OVERLAP_CHUNKS", None)
                else:
                    os.environ["B200_HCCL_OVERLAP_CHUNKS"] = chunks
                for _ in range(3):
                    ksplit_step()
                torch.cuda.synchronize()
                res[label] = round(timed(ksplit_step, 5, world, dev) / (5 * 4) * 1e3, 2)
            os.environ.pop("B200_HCCL_OVERLAP_CHUNKS", None)
            sharded["ksplit_allreduce_w8a8_m4096"] = {
                "plain_us_per_call": res["plain"], "overlapped_us_per_call": res["overlapped"],
                "what": "aclnnQuantMatmulAllReduce, x int8 [4096, 4096/N] @ w int8 [4096/N, 14336] -> bf16 [4096, 14336] summed over "
                        "the ranks by HcclAllReduce (NCCL); overlapped = B200_HCCL_OVERLAP_CHUNKS=2: all-reduce of chunk i on a second "
                        "stream beside the matmul of chunk i+1 (off by default: it measures slower); direct calls, no graph"}
            del qx, qw, qo
        except Exception as e:
            sharded["ksplit_allreduce_w8a8_m4096"] = {"error": repr(e)[:200]}
        torch.cuda.empty_cache()

    # End to end through the C ABI with host buffers: every call's activations come from pinned host memory and
    # every call's result goes back to pinned host memory inside the step; weights stay resident.
    # The loop is a compiled C client of the ABI (cann-on-gpu_b200/csrc/acl_client.c): per call aclrtMemcpyAsync in,
    # phase 1, phase 2, aclrtMemcpyAsync out.  A step is the same `calls` calls as the device-timed step; every call has
    # its own activation and output buffer, the copies travel in groups of E2E_GROUP calls on two copy streams beside the
    # matmuls of the neighbouring groups, and the step ends with everything synchronised.
    E2E_GROUP = int(os.environ.get("B200_BENCH_E2E_GROUP", "15"))
    n = runner.calls_per_step
    hx_all = torch.stack([runner.items[i % ring][-1]["x"].cpu() for i in range(n)]).contiguous().pin_memory()   # [n, M, K]
    hout_all = torch.empty((n, M, ns), dtype=torch.bfloat16).pin_memory()
    dx_all = torch.empty((n, M, K), dtype=torch.bfloat16, device=dev)
    dout_all = torch.empty((n, M, ns), dtype=torch.bfloat16, device=dev)
    tdxs, tdouts = [pkg.AclTensor(dx_all[i]) for i in range(n)], [pkg.AclTensor(dout_all[i]) for i in range(n)]
    client_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libqmm_client.so")
    if not os.path.exists(client_path):
        raise RuntimeError(f"{client_path} is missing: run __graft_entry__.build()")
    client = ctypes.CDLL(client_path)
    client.qmmClientWeightQuantStep.restype = ctypes.c_int
    client.qmmClientWeightQuantStepCapture.restype = ctypes.c_int
    client.qmmClientReplay.restype = ctypes.c_int
    VP = ctypes.c_void_p
    weights = (VP * n)(*[VP(runner.items[i % ring][1].h) for i in range(n)])
    scales = (VP * n)(*[VP(runner.items[i % ring][2].h) for i in range(n)])
    x_tensors = (VP * n)(*[VP(t.h) for t in tdxs])
    out_tensors = (VP * n)(*[VP(t.h) for t in tdouts])
    ws_buf, ws_bytes = runner.ws.get(1, dev)   # the workspace the warm-up calls sized
    # a stream of its own: the legacy default stream cannot be captured
    e2e_stream = torch.cuda.Stream(dev)
    stream = VP(e2e_stream.cuda_stream)
    torch.cuda.synchronize()
    step_args = (ctypes.c_int(n), ctypes.c_int(E2E_GROUP), VP(hx_all.data_ptr()), ctypes.c_size_t(M * K * 2), VP(dx_all.data_ptr()),
                 x_tensors, weights, scales, None, None, ctypes.c_int64(GROUP), out_tensors, VP(dout_all.data_ptr()),
                 VP(hout_all.data_ptr()), ctypes.c_size_t(M * ns * 2), VP(ws_buf.data_ptr()), ctypes.c_uint64(ws_bytes), stream)

    def e2e_direct():
        st = client.qmmClientWeightQuantStep(*step_args)
        if st != 0:
            raise RuntimeError(f"end-to-end client step -> {st}")

    # the step once directly (first launches set kernel attributes), then captured into a model
    # (aclmdlRICaptureBegin / End) and replayed: every replay re-issues all copies and kernels
    e2e_direct()
    model = VP()
    st = client.qmmClientWeightQuantStepCapture(*step_args, ctypes.byref(model))
    if st != 0 or not model.value:
        raise RuntimeError(f"end-to-end client capture -> {st}")

    def e2e_step():
        st = client.qmmClientReplay(model, stream)
        if st != 0:
            raise RuntimeError(f"end-to-end client replay -> {st}")

    with torch.cuda.stream(e2e_stream):   # the timing events go to the stream the step runs on
        for _ in range(args.warmup):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps, world, dev)
        ms_e2e_direct = timed(e2e_direct, max(3, args.steps // 4), world, dev) * args.steps / max(3, args.steps // 4)
    lib.aclmdlRIDestroy(model)
    # the results that came back are the device-timed path's results (same calls, same weights)
    torch.cuda.synchronize()
    if not torch.equal(hout_all[n - 1], runner.out.cpu()) and rank == 0:   # the last call of either step uses the ring's last set
        sys.stderr.write("warning: end-to-end output differs from the device-timed call's output\n")
    v_captured, v_direct = calls * WEIGHT_BYTES / ms_e2e / 1e6, calls * WEIGHT_BYTES / ms_e2e_direct / 1e6
    e2e = {"value": round(max(v_captured, v_direct), 2), "unit": "GB/s",
           "form": "captured step replayed" if v_captured >= v_direct else "step issued call by call from the host",
           "captured_value": round(v_captured, 2),
           "h2d_bytes_per_step": n * M * K * 2, "d2h_bytes_per_step": n * M * ns * 2,
           "host_loop": f"compiled C client of the ABI: a step of {n} calls, each with its own activation buffer copied in from pinned host "
                        f"memory and its own result copied back (aclrtMemcpyAsync in groups of {E2E_GROUP} calls on two copy streams beside "
                        "the matmuls), phase 1 and phase 2 per call, every step synchronised; timed both issued call by call from the host "
                        "and captured once (aclmdlRICaptureBegin/End) and replayed: value is the faster of the two (form)",
           "uncaptured_value": round(v_direct, 2)}

    if rank == 0:
        per_call_ms = ms / calls
        # roofline of the dominant kernel, per launch, on what one GPU streams
        algo = ALGO_BYTES if world == 1 else (K * ns // 2 + (K // GROUP) * ns * 2 + M * K * 2 + M * ns * 2)
        achieved = algo / per_call_ms / 1e6
        traffic, rec = ncu_traffic()
        line = {
            "metric": "w4a16_g128_weight_stream", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "K": K, "N": N, "group": GROUP, "calls_per_step": runner.calls_per_step,
                       "weight_format": "int4 pre-packed once at load time by aclnnTransMatmulWeight into the on-device tile format "
                                        "(ACL_FORMAT_FRACTAL_NZ tensor), resident in HBM; the call is aclnnWeightQuantBatchMatmulV2Ex",
                       "launch": f"one CUDA graph per step ({passes} passes over the ring), replayed",
                       "cache": f"ring of {ring} distinct weight sets per GPU ({ring * (K * ns // 2) >> 20} MiB) larger than 2x L2",
                       "parallelism": (f"N-shard x{world}: rank r owns columns [r*{ns}, (r+1)*{ns}) of the fixed layer, no collective"
                                       if world > 1 else "one GPU, whole layer")},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": traffic if world == 1 else None, "peak_source": pk["source"],
                         "algorithmic_bytes_per_launch": algo, "us_per_call": round(per_call_ms * 1e3, 3),
                         "traffic_record": rec if world == 1 else "captured on the whole layer (one GPU) only"},
            "tflops": round(calls * 2 * M * K * N / ms / 1e9, 3),
            "caller_layout": {"value": round(calls * WEIGHT_BYTES / ms_nd / 1e6, 2), "us_per_call": round(ms_nd / calls * 1e3, 3),
                              "frac": round(algo / (ms_nd / calls) / 1e6 / pk["hbm_gbs"], 4),
                              "what": "the same calls on weights left in the caller's [K,N] layout (2-D TMA boxes at the row pitch) "
                                      "instead of the pre-packed on-device format"},
            "sharded": sharded,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        if world == 1 and not args.no_sweep:
            del runner
            torch.cuda.empty_cache()
            line["sweep"] = sweep(pkg, workloads, dev, pk, with_ref=not args.no_ref_cuda)
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


class WeakRunner(Runner):
    """Runner over whole-layer weight sets (every rank all 28672 columns)."""

    def __init__(self, pkg, sets, dev, passes):
        self.pkg, self.dev, self.passes, self.gather = pkg, dev, passes, None
        self.out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        self.t_out = pkg.AclTensor(self.out)
        self.items = [(pkg.AclTensor(d["x"]), pkg.AclTensor(d["w"], pkg.ACL_INT4, (K, N)), pkg.AclTensor(d["scale"]), None, None, d)
                      for d in sets]
        self.ws = pkg.Workspace()


if __name__ == "__main__":
    main()
