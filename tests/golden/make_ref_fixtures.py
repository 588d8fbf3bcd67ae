"""Records the outputs of the reference's own CUDA backend (oracle/_ref/libascendcl_ref.so, built
by oracle/build_ref.sh from the reference's sources) on a B200 for the cases in cases.py.

Run on a GPU box from the repository root:
    python tests/golden/make_ref_fixtures.py <out.npz>    (then copy it to tests/golden/ref_b200_outputs.npz)
The resulting file is committed as tests/golden/ref_b200_outputs.npz; the tests replay the same
seeded inputs through the CPU checker (pinning it) and through this library's kernels.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import __graft_entry__ as ge  # noqa: E402
import cases  # noqa: E402

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libascendcl_ref.so")


def bits(t):
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main(out_path):
    pkg = ge.load_package()
    from cann_on_gpu_b200 import workloads
    dev = torch.device("cuda:0")
    res = {}
    with pkg.use_library(REF_LIB):
        for name, (gen, kw) in cases.WQ_CASES.items():
            d = getattr(workloads, gen)(**kw)
            out = pkg.weight_quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev),
                                          d["offset"].to(dev) if d["offset"] is not None else None,
                                          int4=d["int4"], name="aclnnWeightQuantBatchMatmul")
            torch.cuda.synchronize()
            res[name] = bits(out)
        for name, kw in cases.QMM_CASES.items():
            d = workloads.w8a8(**kw)
            ws = pkg.Workspace()
            out = pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), out_dtype=kw["out_dtype"],
                                   name="aclnnQuantMatmul", workspace=ws)
            torch.cuda.synchronize()
            res[name] = bits(out)
            # the reference leaves its int32 accumulators in the caller's workspace at byte offset N*K
            M, K, N = d["M"], d["K"], d["N"]
            acc = ws.buf[N * K: N * K + 4 * M * N].clone().view(torch.int32).reshape(M, N)
            res[name + "_acc"] = acc.cpu().numpy()
        for name, (entry, kw) in cases.MX_CASES.items():
            d = workloads.mx(**kw)
            ak = pkg.ACL_FLOAT4_E2M1 if kw["a_fp4"] else pkg.ACL_FLOAT8_E4M3FN
            bk = pkg.ACL_FLOAT4_E2M1 if kw["b_fp4"] else pkg.ACL_FLOAT8_E4M3FN
            out = pkg.mx_matmul(d["a"].reshape(-1).to(dev), ak, d["sa"].to(dev), d["b"].reshape(-1).to(dev), bk,
                                d["sb"].to(dev), d["M"], d["K"], d["N"], out_dtype=torch.float32, name=entry)
            torch.cuda.synchronize()
            res[name] = bits(out)
        x = cases.cast_input().to(dev)
        res["cast_e2m1"] = bits(pkg.cast(x, pkg.ACL_FLOAT, pkg.ACL_FLOAT4_E2M1, cases.CAST_N))
        res["cast_e4m3"] = bits(pkg.cast(x * 64, pkg.ACL_FLOAT, pkg.ACL_FLOAT8_E4M3FN, cases.CAST_N))
        torch.cuda.synchronize()
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    np.savez_compressed(out_path, **res)
    print("wrote", out_path, {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "ref_b200_outputs.npz")
