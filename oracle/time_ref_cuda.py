"""Times the reference's own CUDA backend (oracle/_ref/libascendcl_ref.so, built by build_ref.sh
from the reference's sources for sm_100a) and this library on the same B200, on the closest form of
each benchmark configuration that the reference accepts (fp16 activations, per-channel [N] scales,
fp16 outputs, same-kind MX operands: cuda/src/ops/matmul.cu:761-767,802-807,437,491 of the
reference).  Test infrastructure: prints one JSON line per case.

    python oracle/time_ref_cuda.py > ref_cuda_times.jsonl
"""
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libascendcl_ref.so")
pkg = ge.load_package()
from cann_on_gpu_b200 import workloads  # noqa: E402

dev = torch.device("cuda:0")
torch.cuda.set_device(dev)


def time_calls(make_calls, reps):
    """make_calls() -> list of zero-argument callables (one per weight set).  Graph replay when the
    library's calls can be captured, eager calls otherwise."""
    calls = make_calls()
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


def wq_case(M, K, N, int4, ring):
    def make():
        ws = pkg.Workspace()
        calls = []
        for i in range(ring):
            d = (workloads.w4a16(M=M, K=K, N=N, dtype=torch.float16, per_channel=True, with_bias=False, seed=3000 + i) if int4
                 else workloads.w8a16(M=M, K=K, N=N, dtype=torch.float16, with_offset=True, seed=3000 + i))
            out = torch.empty((M, N), dtype=torch.float16, device=dev)
            args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev), pkg.ACL_INT4 if int4 else pkg.ACL_INT8, (K, N)),
                    pkg.AclTensor(d["scale"].to(dev)), pkg.AclTensor(d["offset"].to(dev)), pkg.AclTensor(out)]
            calls.append(lambda a=args: pkg.call("aclnnWeightQuantBatchMatmul", *a, workspace=ws, device=dev))
        return calls
    return make


def qmm_case(M, K, N, ring):
    def make():
        ws = pkg.Workspace()
        calls = []
        for i in range(ring):
            d = workloads.w8a8(M=M, K=K, N=N, seed=3100 + i, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
            out = torch.empty((M, N), dtype=torch.float16, device=dev)
            args = [pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev)), pkg.AclTensor(out)]
            calls.append(lambda a=args: pkg.call("aclnnQuantMatmul", *a, workspace=ws, device=dev))
        return calls
    return make


def mx_case(M, K, N, fp4, entry):
    def make():
        ws = pkg.Workspace()
        d = workloads.mx(M=M, K=K, N=N, a_fp4=fp4, b_fp4=fp4, seed=3200)
        kind = pkg.ACL_FLOAT4_E2M1 if fp4 else pkg.ACL_FLOAT8_E4M3FN
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
        args = [pkg.AclTensor(d["a"].reshape(-1).to(dev), kind, (M, K)), pkg.AclTensor(d["sa"].to(dev), pkg.ACL_FLOAT8_E8M0, (M, K // 32)),
                pkg.AclTensor(d["b"].reshape(-1).to(dev), kind, (K, N)), pkg.AclTensor(d["sb"].to(dev), pkg.ACL_FLOAT8_E8M0, (K // 32, N)),
                pkg.AclTensor(out)]
        return [lambda a=args: pkg.call(entry, *a, workspace=ws, device=dev)]
    return make


CASES = [
    ("cfg0 W8A16 M=1 K=1024 N=3072 fp16 per-channel", wq_case(1, 1024, 3072, False, 32), 2 * 1024 * 3072, 1024 * 3072, 20),
    ("cfg1-like W4A16 M=1 K=4096 N=4096 fp16 per-channel", wq_case(1, 4096, 4096, True, 16), 2 * 4096 * 4096, 4096 * 4096 // 2, 10),
    ("cfg1-like W4A16 M=16 K=4096 N=4096 fp16 per-channel", wq_case(16, 4096, 4096, True, 16), 2 * 16 * 4096 * 4096, 4096 * 4096 // 2, 5),
    ("cfg1-like W4A16 M=128 K=4096 N=4096 fp16 per-channel", wq_case(128, 4096, 4096, True, 16), 2 * 128 * 4096 * 4096, 4096 * 4096 // 2, 5),
    ("cfg4-like W4A16 M=1 K=8192 N=28672 fp16 per-channel", wq_case(1, 8192, 28672, True, 3), 2 * 8192 * 28672, 8192 * 28672 // 2, 3),
    ("cfg4-like W4A16 M=512 K=8192 N=28672 fp16 per-channel", wq_case(512, 8192, 28672, True, 2), 2 * 512 * 8192 * 28672, 8192 * 28672 // 2, 3),
    ("cfg2-like W8A8 M=8 K=4096 N=14336 fp16 scale/out", qmm_case(8, 4096, 14336, 4), 2 * 8 * 4096 * 14336, 4096 * 14336, 5),
    ("cfg2-like W8A8 M=2048 K=4096 N=14336 fp16 scale/out", qmm_case(2048, 4096, 14336, 2), 2 * 2048 * 4096 * 14336, 4096 * 14336, 5),
    ("cfg3-like MXFP8xMXFP8 4096x8192x8192 (Hw entry)", mx_case(4096, 8192, 8192, False, "aclnnMatmulMxFp8Hw"), 2 * 4096 * 8192 * 8192, 8192 * 8192, 3),
    ("cfg3-like MXFP4xMXFP4 4096x8192x8192 (Hw entry)", mx_case(4096, 8192, 8192, True, "aclnnMatmulMxFp4Hw"), 2 * 4096 * 8192 * 8192, 8192 * 8192 // 2, 3),
]


def main():
    have_ref = os.path.exists(REF_LIB)
    for name, make, flops, wbytes, reps in CASES:
        row = {"case": name}
        for label, lib in (("reference_cuda", REF_LIB if have_ref else None), ("this_library", pkg.LIB_PATH)):
            if lib is None:
                row[label] = "unavailable: oracle/_ref not built"
                continue
            try:
                with pkg.use_library(lib):
                    us, mode = time_calls(make, reps)
                row[label] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "weight_gbs": round(wbytes / us / 1e3, 1),
                              "launch": mode}
            except Exception as e:
                row[label] = "failed: " + repr(e)[:160]
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
