"""Per-CTA time stamps of the decode kernel (csrc/wq_mma.cu compiled with -DWQ_MMA_PROFILE).

Developer aid, not part of the product path: builds a second copy of the library with the stamps compiled
in (lib/libascendcl_profile.so; the normal build has none), runs W4A16 group-128 decode calls back to back
from a CUDA graph over a ring of weight sets larger than L2, and prints, for the LAST call of a replay, when
each phase was reached across the CTAs (microseconds after the first CTA's entry; the previous call's tail
overlaps the start).  Usage, on a B200, from the repository root:

    python cann-on-gpu_b200/decode_profile.py [--build-only | M,N,packed ...]      e.g.  1,28672,1  1,3584,1

K is 8192; packed = 1 uses the on-device weight format, 0 the caller's [K,N] layout.
"""
import ctypes
import importlib.util
import os
import statistics
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PROFILE_LIB = os.path.join(HERE, "lib", "libascendcl_profile.so")
K = 8192
PHASES = ("entry", "barriers ready", "weight producer past its dependency wait", "first stage full", "last stage multiplied",
          "reducer has the last partial tile", "reducer done")


def build_profile_library():
    """The objects of the normal build, with wq_mma.cu recompiled with the stamps (skipped when the profiling library
    is newer than every kernel source; `--build-only` stops after this step, e.g. on a machine without a GPU)."""
    src_dir = os.path.join(HERE, "csrc")
    newest = max(os.path.getmtime(os.path.join(src_dir, f)) for f in os.listdir(src_dir))
    if os.path.exists(PROFILE_LIB) and os.path.getmtime(PROFILE_LIB) >= newest:
        return
    subprocess.run(["make", "-C", HERE, "-j8"], check=True, stdout=subprocess.DEVNULL)
    obj = os.path.join(HERE, "build", "wq_mma_profile.o")
    arch = ["-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(["nvcc", *arch, "-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                    "-I" + os.path.join(HERE, "..", "include"), "-I" + os.path.join(HERE, "csrc"), "--expt-relaxed-constexpr",
                    "-DWQ_MMA_PROFILE", "-c", os.path.join(HERE, "csrc", "wq_mma.cu"), "-o", obj], check=True, stderr=subprocess.DEVNULL)
    others = [os.path.join(HERE, "build", f) for f in sorted(os.listdir(os.path.join(HERE, "build")))
              if f.endswith(".o") and f not in ("wq_mma.o", "wq_mma_profile.o")]
    subprocess.run(["nvcc", *arch, "-shared", "-cudart", "static", "-o", PROFILE_LIB, obj, *others], check=True)


def main(specs):
    if specs and specs[0] == "--build-only":
        build_profile_library()
        return
    import torch
    spec = importlib.util.spec_from_file_location("cann_on_gpu_b200", os.path.join(HERE, "__init__.py"), submodule_search_locations=[HERE])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules["cann_on_gpu_b200"] = pkg
    spec.loader.exec_module(pkg)
    build_profile_library()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    with pkg.use_library(PROFILE_LIB):
        lib = pkg.load(PROFILE_LIB)
        for text in specs:
            M, N, packed = [int(v) for v in text.split(",")]
            nsets = max(3, int(400e6 // (K * N // 2)))
            sets, keep = [], []
            for _ in range(nsets):
                x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(dev)
                w = torch.randint(0, 256, (K * N // 2,), generator=g, dtype=torch.uint8).to(dev)
                sc = (torch.rand((K // 128, N), generator=g) * 0.01).to(torch.bfloat16).to(dev)
                out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
                if packed:
                    w = pkg.pack_weight_nz(w, K, N)
                    tw = pkg.AclTensor(w, pkg.ACL_INT4, (K, N), fmt=pkg.ACL_FORMAT_FRACTAL_NZ, storage=(w.numel() * 2,))
                else:
                    tw = pkg.AclTensor(w, pkg.ACL_INT4, (K, N))
                keep.append((x, w, sc, out))
                sets.append([pkg.AclTensor(x), tw, pkg.AclTensor(sc), None, None, ctypes.c_int64(128), pkg.AclTensor(out)])
            ws = pkg.Workspace()

            def step():
                for a in sets:
                    pkg.call("aclnnWeightQuantBatchMatmulV2Ex", *a, workspace=ws, device=dev)
            step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (20 * nsets)
            buf = (ctypes.c_ulonglong * (8 * 160))()
            lib.aclnnB200DecodeProfile(buf)          # clears the accumulating rows
            graph.replay()
            torch.cuda.synchronize()
            lib.aclnnB200DecodeProfile(buf)
            ctas = sum(1 for c in range(160) if buf[c])
            rows = [[buf[r * 160 + c] for c in range(ctas)] for r in range(8)]
            t0 = min(rows[0])
            print(f"M={M} K={K} N={N} packed={packed}: {us:.2f} us per call back to back (profiling build), {ctas} CTAs")
            for r, name in enumerate(PHASES):
                v = [(t - t0) / 1e3 for t in rows[r] if t]
                print(f"    {name:44s} min {min(v):6.2f}  median {statistics.median(v):6.2f}  max {max(v):6.2f}")
            v = [t / 1e3 / nsets for t in rows[7]]
            print(f"    reducer time spent on tiles shared between CTAs, per call: median {statistics.median(v):.2f}  max {max(v):.2f} us")


if __name__ == "__main__":
    main(sys.argv[1:] or ["1,28672,1"])
