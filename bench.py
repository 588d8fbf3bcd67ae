"""Benchmark of the quantized-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-sweep]

Workload (config.workload): W4A16 group-wise weight-only matmul, x bf16 [M=16, K=4096] @ int4
[4096, 4096] with bf16 scales and offsets per 128 rows of K and a bf16 bias -- the decode-shaped,
HBM-bound case of the benchmark configurations.  One step is one pass of the operator over a ring
of R distinct weight sets whose total size exceeds twice the L2, so every call streams its weights
from HBM.  The metric is weight GB/s: packed weight bytes streamed per second, summed over ranks.

With N > 1 (launched by torch.distributed.run) every rank owns one column shard of that size of a
[4096, 4096*N] layer and runs it independently: no data-path collective, weak scaling.

--impl reference times the CPU restatement of the reference's algorithm (oracle/) on the host cores
for the same operator.  Synthetic seeded inputs throughout.
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

M, K, N, GROUP = 16, 4096, 4096, 128
RING = 32  # 32 x 8.4 MB of packed weights = 268 MB > 2 x 126 MB of L2
WEIGHT_BYTES = K * N // 2
# Algorithmic bytes of one call: packed weights + scales + offsets + activations + output + bias.
ALGO_BYTES = WEIGHT_BYTES + 2 * (K // GROUP) * N * 2 + M * K * 2 + M * N * 2 + N * 2


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
        d = workloads.w4a16(M=M, K=K, N=N, group=GROUP, seed=1001 + 1000 * rank + i)
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
                               pkg.AclTensor(d["offset"]), pkg.AclTensor(d["bias"]), d))
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


def sweep(pkg, workloads, dev, pk):
    """Other configurations, timed per call with CUDA events (not part of the headline value)."""
    rows = []

    def time_calls(fn, flops, wbytes, name, reps=20, ring=1):
        for _ in range(3):
            fn(0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for r in range(reps):
            fn(r % ring)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        rows.append({"case": name, "ms": round(ms, 5), "tflops": round(flops / ms / 1e9, 2),
                     "weight_gbs": round(wbytes / ms / 1e6, 1)})

    try:
        # config 0: W8A16 M=1 K=1024 N=3072 (3 MB: L2-resident and launch-bound; 64 distinct weight sets)
        sets = [workloads.w8a16(seed=1000 + i) for i in range(64)]
        ds = [{k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items()} for d in sets]
        time_calls(lambda i: pkg.weight_quant_matmul(ds[i]["x"], ds[i]["w"], ds[i]["scale"], name="aclnnWeightQuantBatchMatmulV2"),
                   2 * 1024 * 3072, 1024 * 3072, "cfg0 W8A16 M=1 K=1024 N=3072", reps=128, ring=64)
        del ds
        # config 1 at M = 1 and 128 over the same ring idea (16 sets)
        for m in (1, 128):
            sets = [workloads.w4a16(M=m, seed=1001 + i) for i in range(16)]
            ds = [{k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items() if k != "w_vals"} for d in sets]
            time_calls(lambda i: pkg.weight_quant_matmul(ds[i]["x"], ds[i]["w"], ds[i]["scale"], ds[i]["offset"], ds[i]["bias"],
                                                         int4=True, group=GROUP),
                       2 * m * K * N, WEIGHT_BYTES, f"cfg1 W4A16 g128 M={m} K=4096 N=4096", reps=64, ring=16)
            del ds
        # config 2: W8A8 M=2048 K=4096 N=14336
        for m in (8, 2048):
            d = workloads.w8a8(M=m)
            dd = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items()}
            time_calls(lambda i: pkg.quant_matmul(dd["x"], dd["w"], dd["scale"], dd["pertoken"], dd["bias"]),
                       2 * m * 4096 * 14336, 4096 * 14336, f"cfg2 W8A8 M={m} K=4096 N=14336", reps=10)
            del dd
        # config 3: MXFP8 x MXFP4 4096 x 8192 x 8192
        d = workloads.mx()
        a, b, sa, sb = d["a"].reshape(-1).to(dev), d["b"].reshape(-1).to(dev), d["sa"].to(dev), d["sb"].to(dev)
        time_calls(lambda i: pkg.mx_matmul(a, pkg.ACL_FLOAT8_E4M3FN, sa, b, pkg.ACL_FLOAT4_E2M1, sb, 4096, 8192, 8192),
                   2 * 4096 * 8192 * 8192, 8192 * 8192 // 2, "cfg3 MXFP8xMXFP4 M=4096 K=8192 N=8192", reps=5)
    except Exception as e:  # a sweep failure must not lose the headline line
        rows.append({"error": repr(e)[:200]})
    for r in rows:
        if "tflops" in r:
            r["frac_hbm"] = round(r["weight_gbs"] / pk["hbm_gbs"], 3)
            r["frac_bf16_burst"] = round(r["tflops"] / pk["bf16_tflops"], 3)
    return rows


def cpu_baseline(seconds=12.0):
    """The CPU restatement (BLAS-backed form) of the same operator on the host cores."""
    o = ge.load_oracle()
    ge.load_package()
    from cann_on_gpu_b200 import workloads
    d = workloads.w4a16(M=M, K=K, N=N, group=GROUP, seed=1001)
    args = (d["x"].float().numpy(), d["w"].numpy(), True, d["scale"].float().numpy(), d["offset"].float().numpy(),
            d["bias"].float().numpy(), M, K, N, GROUP)
    o.wqbmm_fast(*args)
    n, t0 = 0, time.perf_counter()
    while True:
        o.wqbmm_fast(*args)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or n >= 200:
            break
    return {"value": round(n * WEIGHT_BYTES / dt / 1e9, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n} passes of the numpy/BLAS restatement over one 4096x4096 int4 weight set at M=16 ({dt:.1f} s)"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    o = ge.load_oracle()
    ge.load_package()
    from cann_on_gpu_b200 import workloads
    d = workloads.w4a16(M=M, K=K, N=N, group=GROUP, seed=1001)
    a = (d["x"].float().numpy(), d["w"].numpy(), True, d["scale"].float().numpy(), d["offset"].float().numpy(),
         d["bias"].float().numpy(), M, K, N, GROUP)
    for _ in range(max(1, args.warmup)):
        o.wqbmm_fast(*a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.wqbmm_fast(*a)
    dt = time.perf_counter() - t0
    v = args.steps * WEIGHT_BYTES / dt / 1e9
    sample = f"each step = 1 of the {RING} weight sets of the device arm's step (one 4096x4096 int4 matrix at M=16)"
    print(json.dumps({
        "impl": "reference", "metric": "w4a16_g128_weight_stream", "value": round(v, 4), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "W4A16 group-128 weight-only matmul, x bf16 [16,4096] @ int4 [4096,4096], bf16 scale+offset+bias",
                   "M": M, "K": K, "N": N, "group": GROUP},
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
    ms = timed(runner.replay, args.steps, world, dev)
    launches = runner.launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    calls = args.steps * args.ring
    value = world * calls * WEIGHT_BYTES / ms / 1e6  # GB/s over all ranks

    # End to end through the C ABI with host buffers: activations come from pinned host memory and
    # the result goes back to pinned host memory on every call; weights stay resident.
    hx = [d["x"].cpu().pin_memory() for *_, d in runner.items]
    hout = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    dx = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
    tdx = pkg.AclTensor(dx)

    def e2e_step():
        for i in range(args.ring):
            dx.copy_(hx[i], non_blocking=True)
            runner.call(i, tdx)
            hout.copy_(runner.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(args.warmup):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps, world, dev)
    e2e = {"value": round(world * calls * WEIGHT_BYTES / ms_e2e / 1e6, 2), "unit": "GB/s",
           "h2d_bytes_per_step": args.ring * M * K * 2, "d2h_bytes_per_step": args.ring * M * N * 2}

    if rank == 0:
        per_call_ms = ms / calls
        achieved = ALGO_BYTES / per_call_ms / 1e6
        line = {
            "metric": "w4a16_g128_weight_stream", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "W4A16 group-128 weight-only matmul, x bf16 [16,4096] @ int4 [4096,4096], bf16 scale+offset+bias",
                       "M": M, "K": K, "N": N, "group": GROUP, "calls_per_step": args.ring,
                       "launch": "one CUDA graph per step (a pass over the ring), replayed",
                       "cache": f"ring of {args.ring} distinct weight sets ({args.ring * WEIGHT_BYTES >> 20} MiB) larger than 2x L2",
                       "parallelism": f"N-shard x{world}, no collective"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": None, "peak_source": pk["source"],
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
