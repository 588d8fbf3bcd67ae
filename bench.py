"""Benchmark of the quantized-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-sweep]

Workload (config.workload): the largest single-GPU configuration of the benchmark set -- the
Llama-70B-shaped gate/up projection as a W4A16 group-wise weight-only matmul, x bf16 [M=1, K=8192] @
int4 [8192, 28672] with bf16 scales per 128 rows of K (117 MB of packed weights per call, decode
shape, HBM-bound).  The smaller W4A16 configuration (4096 x 4096, 8.4 MB) fits in L2 and its ideal
time of 1.3 us is below a kernel launch, so it cannot show a memory roofline; it is reported in the
sweep instead.  One step is one pass of the operator over a ring of R distinct weight sets whose
total size exceeds twice the L2, so every call streams its weights from HBM.  The metric is weight
GB/s: packed weight bytes streamed per second, summed over ranks.

With N > 1 (launched by torch.distributed.run) every rank owns one 28672-column shard of a
[8192, 28672*N] layer and runs it independently: no data-path collective, weak scaling.

--impl reference times the CPU restatement of the reference's algorithm (oracle/) on the host cores
for the same operator, on a column slice of the weight.  Synthetic seeded inputs throughout.
"""
import argparse
import ctypes
import json
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
RING = 3  # 3 x 117 MB of packed weights = 352 MB > 2 x 126 MB of L2
WEIGHT_BYTES = K * N // 2
# Algorithmic bytes of one call: packed weights + group scales + activations + output.
ALGO_BYTES = WEIGHT_BYTES + (K // GROUP) * N * 2 + M * K * 2 + M * N * 2
WORKLOAD = ("W4A16 group-128 weight-only matmul, Llama-70B gate/up shape: x bf16 [1,8192] @ int4 [8192,28672], "
            "bf16 group scales, no offset, no bias")
CPU_SLICE_N = 2048  # columns of the weight the CPU legs work on
# DRAM bytes (read + write) of one launch of the dominant kernel on this workload, from the ncu capture
# summarised in profiles/wq_mma_kernel_w4a16_llama_gateup_m1.md.
NCU_TRAFFIC_BYTES = 124_836_608


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


def make_ring(workloads, dev, rank, ring):
    """`ring` weight sets (distinct seeds) resident on the device, plus the shared activations."""
    sets = []
    for i in range(ring):
        d = workloads.w4a16(M=M, K=K, N=N, group=GROUP, seed=1004 + 1000 * rank + i, with_offset=False, with_bias=False)
        sets.append({k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items() if k != "w_vals"})
    return sets


class Runner:
    """Pre-built aclTensor handles for the ring so the timed loop is phase 1 + phase 2 only."""

    def __init__(self, pkg, sets, dev):
        self.pkg, self.dev = pkg, dev
        self.out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        self.t_out = pkg.AclTensor(self.out)
        self.items = []
        for d in sets:
            self.items.append((pkg.AclTensor(d["x"]), pkg.AclTensor(d["w"], pkg.ACL_INT4, (K, N)), pkg.AclTensor(d["scale"]),
                               None, None, d))
        self.ws = pkg.Workspace()

    def call(self, i, x_handle=None):
        tx, tw, ts, to, tb, _ = self.items[i]
        self.pkg.call("aclnnWeightQuantBatchMatmulV2Ex", x_handle or tx, tw, ts, to, tb, ctypes.c_int64(GROUP), self.t_out,
                      workspace=self.ws, device=self.dev)

    def step(self):
        for i in range(len(self.items)):
            self.call(i)

    def capture(self):
        """One step (a pass over the ring) as a CUDA graph: phase 2 neither allocates nor synchronises,
        so the calls can be captured; replaying removes the host's per-call overhead from the timing."""
        self.graph = torch.cuda.CUDAGraph()
        lib = self.pkg.load()
        n0 = lib.aclnnB200KernelLaunchCount()
        with torch.cuda.graph(self.graph):
            self.step()
        self.launches_per_step = lib.aclnnB200KernelLaunchCount() - n0

    def replay(self):
        self.graph.replay()


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


def sweep(pkg, workloads, dev, pk, only=None):
    """The other benchmark configurations: each case is captured as one CUDA graph over a ring of
    distinct weight sets (larger than L2 where memory allows) and timed with CUDA events."""
    rows = []

    def wanted(name):
        return only is None or only in name

    def run_case(name, calls, flops, wbytes, reps):
        # calls: list of zero-argument functions, one per weight set of the ring
        ws = pkg.Workspace()
        for c in calls:
            c(ws)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for c in calls:
                c(ws)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * len(calls))
        rows.append({"case": name, "us": round(ms * 1e3, 2), "tflops": round(flops / ms / 1e9, 2),
                     "weight_gbs": round(wbytes / ms / 1e6, 1), "ring": len(calls)})

    def wq_calls(sets, int4, group, ex=True):
        calls = []
        for d in sets:
            k, n = d["K"], d["N"]
            out = torch.empty((d["M"], n), dtype=d["x"].dtype, device=dev)
            args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev), pkg.ACL_INT4 if int4 else pkg.ACL_INT8, (k, n)),
                    pkg.AclTensor(d["scale"].to(dev)), pkg.AclTensor(d["offset"].to(dev)) if d["offset"] is not None else None,
                    pkg.AclTensor(d["bias"].to(dev)) if d["bias"] is not None else None, ctypes.c_int64(group), pkg.AclTensor(out)]
            calls.append(lambda ws, a=args: pkg.call("aclnnWeightQuantBatchMatmulV2Ex", *a, workspace=ws, device=dev))
        return calls

    if only is not None and only.startswith("case:"):
        # one custom case, e.g. --sweep-only case:w4,128,8192,28672,128  (kind w4 | w8 | i8, M, K, N[, group])
        kind, m, k, n, *rest = only[5:].split(",")
        m, k, n = int(m), int(k), int(n)
        group = int(rest[0]) if rest else 128
        wb = k * n // 2 if kind == "w4" else k * n
        ring = max(2, min(32, 300_000_000 // wb + 1))
        if kind in ("w4", "w8"):
            gen = workloads.w4a16 if kind == "w4" else workloads.w8a16
            kw = dict(group=group, with_offset=False, with_bias=False) if kind == "w4" else dict(dtype=torch.bfloat16)
            sets = [gen(M=m, K=k, N=n, seed=1100 + i, **kw) for i in range(ring)]
            run_case(f"{kind} M={m} K={k} N={n} group={sets[0]['group']} bf16", wq_calls(sets, kind == "w4", sets[0]["group"]),
                     2 * m * k * n, wb, 5)
        else:
            calls = []
            for i in range(ring):
                d = workloads.w8a8(M=m, K=k, N=n, seed=1100 + i)
                out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev)), None,
                        pkg.AclTensor(d["pertoken"].to(dev)), pkg.AclTensor(d["bias"].to(dev)), pkg.AclTensor(out)]
                calls.append(lambda ws, a=args: pkg.call("aclnnQuantMatmulV4Ex", *a, workspace=ws, device=dev))
            run_case(f"W8A8 M={m} K={k} N={n} bf16 out", calls, 2 * m * k * n, wb, 5)
        only = "\0"   # nothing else
    try:
        # config 0: W8A16 M=1 K=1024 N=3072 (3 MB per call: L2-resident and launch-bound)
        if wanted("cfg0 W8A16 per-channel M=1 K=1024 N=3072 fp16"):
            sets = [workloads.w8a16(seed=1000 + i) for i in range(32)]
            run_case("cfg0 W8A16 per-channel M=1 K=1024 N=3072 fp16", wq_calls(sets, False, 0), 2 * 1024 * 3072, 1024 * 3072, 20)
        # config 1: W4A16 g128 K=4096 N=4096 with offset and bias, M = 1 / 16 / 128 (8.4 MB per call)
        for m in (1, 16, 128):
            name = f"cfg1 W4A16 g128 M={m} K=4096 N=4096 bf16 +offset +bias"
            if not wanted(name):
                continue
            sets = [workloads.w4a16(M=m, seed=1001 + i) for i in range(32)]
            run_case(name, wq_calls(sets, True, 128), 2 * m * 4096 * 4096, 4096 * 4096 // 2, 10)
            del sets
        # config 4: Llama-70B shapes, W4A16 g128, no offset
        for which, k, n in (("gate/up", 8192, 28672), ("down", 28672, 8192)):
            for m in ((32, 512, 4096) if which == "gate/up" else (32,)):
                name = f"cfg4 W4A16 g128 {which} M={m} K={k} N={n} bf16"
                if not wanted(name):
                    continue
                sets = [workloads.llama70b_shard(m, "gate_up" if which == "gate/up" else "down", seed=1004 + i) for i in range(3)]
                run_case(name, wq_calls(sets, True, 128), 2 * m * k * n, k * n // 2, 5 if m < 4096 else 3)
                del sets
        # config 2: W8A8 K=4096 N=14336, per-token x per-channel scales, int32 bias, bf16 out
        for m in (1, 8, 256, 2048, 4096):
            if not wanted(f"cfg2 W8A8 M={m} K=4096 N=14336 bf16 out"):
                continue
            calls = []
            for i in range(5):
                d = workloads.w8a8(M=m, seed=1002 + i)
                out = torch.empty((m, 14336), dtype=torch.bfloat16, device=dev)
                args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev)), None,
                        pkg.AclTensor(d["pertoken"].to(dev)), pkg.AclTensor(d["bias"].to(dev)), pkg.AclTensor(out)]
                calls.append(lambda ws, a=args: pkg.call("aclnnQuantMatmulV4Ex", *a, workspace=ws, device=dev))
            run_case(f"cfg2 W8A8 M={m} K=4096 N=14336 bf16 out", calls, 2 * m * 4096 * 14336, 4096 * 14336, 5)
            del calls
        # the activation quantiser in front of config 2 (HBM-bound: "weight_gbs" here is all bytes moved,
        # rows * D * (2 + 1) + rows * 4, per second)
        for m in (2048, 4096):
            name = f"DynamicQuant per-token bf16 [{m},4096] -> int8 (feeds cfg2)"
            if not wanted(name):
                continue
            calls = []
            for i in range(12):   # 12 x (32 MB in + 16 MB out) > 2 x L2
                x = torch.randn((m, 4096), generator=torch.Generator().manual_seed(3000 + i)).to(torch.bfloat16).to(dev)
                q = torch.empty((m, 4096), dtype=torch.int8, device=dev)
                sc = torch.empty((m,), dtype=torch.float32, device=dev)
                args = [pkg.AclTensor(x), pkg.AclTensor(q), pkg.AclTensor(sc)]
                calls.append(lambda ws, a=args: pkg.call("aclnnDynamicQuant", *a, workspace=ws, device=dev))
            run_case(name, calls, 0, m * 4096 * 3 + m * 4, 10)
            del calls
        # SwiGLU + per-token quantiser between a gate/up projection [m, 2 x 14336] and a W8A8 down projection
        # (bytes moved: rows * (2 D * 2 + D) + rows * 4)
        for m in (2048,):
            name = f"SwiGluQuant bf16 [{m},28672] -> int8 [{m},14336]"
            if not wanted(name):
                continue
            calls = []
            for i in range(3):   # 3 x (117 MB in + 29 MB out) > 2 x L2
                x = torch.randn((m, 28672), generator=torch.Generator().manual_seed(3100 + i)).to(torch.bfloat16).to(dev)
                q = torch.empty((m, 14336), dtype=torch.int8, device=dev)
                sc = torch.empty((m,), dtype=torch.float32, device=dev)
                args = [pkg.AclTensor(x), pkg.AclTensor(q), pkg.AclTensor(sc)]
                calls.append(lambda ws, a=args: pkg.call("aclnnSwiGluQuant", *a, workspace=ws, device=dev))
            run_case(name, calls, 0, m * 14336 * 5 + m * 4, 10)
            del calls
        # config 3: MXFP8 x MXFP4 4096 x 8192 x 8192
        if not wanted("cfg3 MXFP8xMXFP4 M=4096 K=8192 N=8192 bf16 out"):
            raise StopIteration
        d = workloads.mx()
        a, b, sa, sb = d["a"].reshape(-1).to(dev), d["b"].reshape(-1).to(dev), d["sa"].to(dev), d["sb"].to(dev)
        out = torch.empty((4096, 8192), dtype=torch.bfloat16, device=dev)
        args = [pkg.AclTensor(a, pkg.ACL_FLOAT8_E4M3FN, (4096, 8192)), pkg.AclTensor(sa, pkg.ACL_FLOAT8_E8M0, (4096, 256)),
                pkg.AclTensor(b, pkg.ACL_FLOAT4_E2M1, (8192, 8192)), pkg.AclTensor(sb, pkg.ACL_FLOAT8_E8M0, (256, 8192)),
                pkg.AclTensor(out)]
        run_case("cfg3 MXFP8xMXFP4 M=4096 K=8192 N=8192 bf16 out",
                 [lambda ws, a_=args: pkg.call("aclnnMatmulMxFp8", *a_, workspace=ws, device=dev)],
                 2 * 4096 * 8192 * 8192, 8192 * 8192 // 2, 3)
    except StopIteration:
        pass
    except Exception as e:  # a sweep failure must not lose the headline line
        rows.append({"error": repr(e)[:300]})
    for r in rows:
        if "tflops" in r:
            r["frac_hbm_measured"] = round(r["weight_gbs"] / pk["hbm_gbs"], 3)
            r["frac_bf16_measured_burst"] = round(r["tflops"] / pk["bf16_tflops"], 3)
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
              f"{RING} weight sets of the device arm's step)")
    print(json.dumps({
        "impl": "reference", "metric": "w4a16_g128_weight_stream", "value": round(v, 4), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M, "K": K, "N": N, "group": GROUP},
        "cpu_baseline": {"value": round(v, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--ring", type=int, default=RING)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--sweep-only", default=None, help="run only the sweep cases whose name contains this text, and nothing else; "
                         "case:<w4|w8|i8>,M,K,N[,group] times one custom shape instead")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
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
        print(json.dumps({"sweep": sweep(pkg, workloads, dev, pk, only=args.sweep_only)}))
        return
    runner = Runner(pkg, make_ring(workloads, dev, rank, args.ring), dev)
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
    calls = args.steps * args.ring
    value = world * calls * WEIGHT_BYTES / ms / 1e6  # GB/s over all ranks

    # End to end through the C ABI with host buffers: activations come from pinned host memory and
    # the result goes back to pinned host memory on every call; weights stay resident.
    hx = [d["x"].cpu().pin_memory() for *_, d in runner.items]
    hout = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    dxs = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    douts = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    tdxs, tdouts = [pkg.AclTensor(t) for t in dxs], [pkg.AclTensor(t) for t in douts]

    # The loop itself is a compiled C client of the ABI (cann-on-gpu_b200/csrc/acl_client.c): per call
    # aclrtMemcpyAsync in, phase 1, phase 2, aclrtMemcpyAsync out, software-pipelined over three streams
    # (two activation and two output buffers), everything synchronised at the end of the pass.
    client_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libqmm_client.so")
    if not os.path.exists(client_path):
        raise RuntimeError(f"{client_path} is missing: run __graft_entry__.build()")
    client = ctypes.CDLL(client_path)
    client.qmmClientWeightQuantPass.restype = ctypes.c_int
    n = args.ring
    VP = ctypes.c_void_p
    host_x = (VP * n)(*[VP(h.data_ptr()) for h in hx])
    weights = (VP * n)(*[VP(it[1].h) for it in runner.items])
    scales = (VP * n)(*[VP(it[2].h) for it in runner.items])
    dev_x = (VP * 2)(*[VP(t.data_ptr()) for t in dxs])
    x_tensors = (VP * 2)(*[VP(t.h) for t in tdxs])
    dev_out = (VP * 2)(*[VP(t.data_ptr()) for t in douts])
    out_tensors = (VP * 2)(*[VP(t.h) for t in tdouts])
    ws_buf, ws_bytes = runner.ws.get(1, dev)   # the workspace the warm-up calls sized
    # a stream of its own: the legacy default stream cannot be captured
    e2e_stream = torch.cuda.Stream(dev)
    stream = VP(e2e_stream.cuda_stream)
    torch.cuda.synchronize()

    def e2e_direct():
        st = client.qmmClientWeightQuantPass(ctypes.c_int(n), host_x, ctypes.c_size_t(M * K * 2), dev_x, x_tensors,
                                             weights, scales, None, None, ctypes.c_int64(GROUP), out_tensors, dev_out,
                                             VP(hout.data_ptr()), ctypes.c_size_t(M * N * 2),
                                             VP(ws_buf.data_ptr()), ctypes.c_uint64(ws_bytes), stream)
        if st != 0:
            raise RuntimeError(f"end-to-end client pass -> {st}")

    # the pass once directly (first launches set kernel attributes), then captured into a model
    # (aclmdlRICaptureBegin / End) and replayed: every replay re-issues all copies and kernels
    e2e_direct()
    client.qmmClientWeightQuantCapture.restype = ctypes.c_int
    client.qmmClientReplay.restype = ctypes.c_int
    model = VP()
    st = client.qmmClientWeightQuantCapture(ctypes.c_int(n), host_x, ctypes.c_size_t(M * K * 2), dev_x, x_tensors, weights, scales,
                                            None, None, ctypes.c_int64(GROUP), out_tensors, dev_out, VP(hout.data_ptr()),
                                            ctypes.c_size_t(M * N * 2), VP(ws_buf.data_ptr()), ctypes.c_uint64(ws_bytes), stream,
                                            ctypes.byref(model))
    if st != 0 or not model.value:
        raise RuntimeError(f"end-to-end client capture -> {st}")

    def e2e_step():
        st = client.qmmClientReplay(model, stream)
        if st != 0:
            raise RuntimeError(f"end-to-end client replay -> {st}")

    with torch.cuda.stream(e2e_stream):   # the timing events go to the stream the pass runs on
        for _ in range(args.warmup):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps, world, dev)
        ms_e2e_direct = timed(e2e_direct, max(3, args.steps // 4), world, dev) * args.steps / max(3, args.steps // 4)
    lib.aclmdlRIDestroy(model)
    e2e = {"value": round(world * calls * WEIGHT_BYTES / ms_e2e / 1e6, 2), "unit": "GB/s",
           "h2d_bytes_per_step": args.ring * M * K * 2, "d2h_bytes_per_step": args.ring * M * N * 2,
           "host_loop": "compiled C client of the ABI: memcpy in, phase 1, phase 2, memcpy out per call, pipelined over three streams, "
                        "captured once (aclmdlRICaptureBegin/End) and replayed per step; all synchronised per step",
           "uncaptured_value": round(world * calls * WEIGHT_BYTES / ms_e2e_direct / 1e6, 2)}

    if rank == 0:
        per_call_ms = ms / calls
        achieved = ALGO_BYTES / per_call_ms / 1e6
        line = {
            "metric": "w4a16_g128_weight_stream", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "K": K, "N": N, "group": GROUP, "calls_per_step": args.ring,
                       "launch": "one CUDA graph per step (a pass over the ring), replayed",
                       "cache": f"ring of {args.ring} distinct weight sets ({args.ring * WEIGHT_BYTES >> 20} MiB) larger than 2x L2",
                       "parallelism": f"N-shard x{world}, no collective"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": NCU_TRAFFIC_BYTES, "peak_source": pk["source"],
                         "algorithmic_bytes_per_launch": ALGO_BYTES, "us_per_call": round(per_call_ms * 1e3, 3)},
            "tflops": round(world * calls * 2 * M * K * N / ms / 1e9, 3),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        if world == 1 and not args.no_sweep:
            del runner
            torch.cuda.empty_cache()
            line["sweep"] = sweep(pkg, workloads, dev, pk)
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
