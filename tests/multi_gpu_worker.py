"""One rank of the two-GPU checks (run by test_multi_gpu.py as `python multi_gpu_worker.py rank world dir`).

Rank r uses GPU r.  The communicator is set up the way an HCCL program does it (tools/mc2_2node.cpp:24-31
of the reference): rank 0 takes HcclGetRootInfo and hands the blob to the others -- here through a file --
then every rank calls HcclCommInitRootInfo.  Checks:
  1. column sharding: each rank multiplies its [K, N/g] shard, HcclAllGather returns [g][M][N/g], the
     interleave is the [M, N] result of the whole problem;
  2. K-split all-reduce forms: aclnnWeightQuantMatmulAllReduce and aclnnQuantMatmulAllReduce sum the
     ranks' partial products;
  3. the same with many rows and B200_HCCL_OVERLAP_CHUNKS set, where the all-reduce of a row chunk overlaps the
     next chunk's matmul.
"""
import ctypes
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as ge  # noqa: E402
from util import assert_close, f32, to_np  # noqa: E402


def main():
    rank, world, tmp = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    pkg = ge.load_package()
    oracle = ge.load_oracle()
    from cann_on_gpu_b200 import workloads
    hccl_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
    pkg.load()
    hccl = pkg.load(hccl_path)

    info = ctypes.create_string_buffer(4108)
    blob = os.path.join(tmp, "root_info.bin")
    if rank == 0:
        assert hccl.HcclGetRootInfo(info) == 0
        with open(blob + ".tmp", "wb") as f:
            f.write(info.raw)
        os.rename(blob + ".tmp", blob)
    else:
        t0 = time.time()
        while not os.path.exists(blob):
            assert time.time() - t0 < 60, "rank 0 never published the root info"
            time.sleep(0.05)
        info.raw = open(blob, "rb").read()
    comm = ctypes.c_void_p()
    assert hccl.HcclCommInitRootInfo(ctypes.c_uint32(world), info, ctypes.c_uint32(rank), ctypes.byref(comm)) == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    # 1. column shards + all-gather
    M = 4
    full = workloads.w4a16(M=M, K=1024, N=1024 * world, group=128, dtype=torch.bfloat16, seed=77)
    mine = workloads.shard_columns(full, world, rank)
    out_r = pkg.weight_quant_matmul(mine["x"].to(dev), mine["w"].to(dev), mine["scale"].to(dev), mine["offset"].to(dev),
                                    mine["bias"].to(dev), int4=True, group=128)
    gathered = torch.empty((world, M, mine["N"]), dtype=torch.bfloat16, device=dev)
    HCCL_BF16 = 11   # HCCL_DATA_TYPE_BFP16 (include/hccl/hccl_types.h)
    assert hccl.HcclAllGather(ctypes.c_void_p(out_r.data_ptr()), ctypes.c_void_p(gathered.data_ptr()),
                              ctypes.c_uint64(out_r.numel()), ctypes.c_int(HCCL_BF16), comm, stream) == 0
    torch.cuda.synchronize()
    whole = workloads.interleave_gathered(gathered, world, M, full["N"])
    ref = oracle.wqbmm_fast(f32(full["x"]), full["w"].numpy(), True, f32(full["scale"]), f32(full["offset"]), f32(full["bias"]),
                            M, full["K"], full["N"], 128)
    assert_close(to_np(whole), ref, f"rank {rank}: gathered column shards")

    # 2. K-split all-reduce forms (reference signatures: fp16, per-channel)
    d = workloads.w8a16(M=8, K=512 * world, N=256, dtype=torch.float16, with_offset=True, seed=78)
    ks = slice(rank * 512, (rank + 1) * 512)
    x_r, w_r = d["x"][:, ks].contiguous().to(dev), d["w"][ks, :].contiguous().to(dev)
    out = torch.empty((8, 256), dtype=torch.float16, device=dev)
    with pkg.use_library(hccl_path):
        pkg.call("aclnnWeightQuantMatmulAllReduce", pkg.AclTensor(x_r), pkg.AclTensor(w_r), pkg.AclTensor(d["scale"].to(dev)),
                 pkg.AclTensor(d["offset"].to(dev)), comm, pkg.AclTensor(out))
    torch.cuda.synchronize()
    ref = oracle.wqbmm_fast(f32(d["x"]), d["w"].numpy(), False, f32(d["scale"]), f32(d["offset"]), None, 8, d["K"], 256, 0)
    assert_close(to_np(out), ref, f"rank {rank}: aclnnWeightQuantMatmulAllReduce")

    q = workloads.w8a8(M=16, K=256 * world, N=128, seed=79, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    ks = slice(rank * 256, (rank + 1) * 256)
    qx, qw = q["x"][:, ks].contiguous().to(dev), q["w"][ks, :].contiguous().to(dev)
    out = torch.empty((16, 128), dtype=torch.float16, device=dev)
    with pkg.use_library(hccl_path):
        pkg.call("aclnnQuantMatmulAllReduce", pkg.AclTensor(qx), pkg.AclTensor(qw), pkg.AclTensor(q["scale"].to(dev)), comm,
                 pkg.AclTensor(out))
    torch.cuda.synchronize()
    acc = oracle.qmm_acc_fast(q["x"].numpy(), q["w"].numpy(), 16, q["K"], 128)
    ref = oracle.qmm_epilogue_fast(acc, f32(q["scale"])).astype(np.float64)
    assert_close(to_np(out), ref, f"rank {rank}: aclnnQuantMatmulAllReduce")

    # the same K-split followed by residual add + RMS norm: the sum over ranks must happen on the
    # partial outputs, before the norm
    g = torch.Generator().manual_seed(81)
    res = torch.randn((16, 128), generator=g).to(torch.float16)
    gamma = (torch.rand(128, generator=g) + 0.5).to(torch.float16)
    y = torch.empty((16, 128), dtype=torch.float16, device=dev)
    rs = torch.empty((16, 128), dtype=torch.float16, device=dev)
    with pkg.use_library(hccl_path):
        pkg.call("aclnnQuantMatmulAllReduceAddRmsNorm", pkg.AclTensor(qx), pkg.AclTensor(qw), pkg.AclTensor(q["scale"].to(dev)),
                 pkg.AclTensor(res.to(dev)), pkg.AclTensor(gamma.to(dev)), ctypes.c_double(1e-5), comm, pkg.AclTensor(y), pkg.AclTensor(rs))
    torch.cuda.synchronize()
    want_y, want_sum = oracle.add_rmsnorm(out.float().cpu().numpy(), f32(res), f32(gamma), 1e-5, "f16")
    assert np.array_equal(rs.float().cpu().numpy(), want_sum), f"rank {rank}: residual sum of the norm matmul"
    assert_close(to_np(y), want_y.astype(np.float64), f"rank {rank}: aclnnQuantMatmulAllReduceAddRmsNorm")

    # 3. many rows: the all-reduce of one row chunk overlaps the matmul of the next (second stream, events);
    # the chunked form must give the bits of the plain sequence, and both the oracle's result
    big = workloads.w8a8(M=1100, K=256 * world, N=512, seed=83, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    bx, bw = big["x"][:, ks].contiguous().to(dev), big["w"][ks, :].contiguous().to(dev)
    outs = {}
    for chunks in ("1", "4", None):     # plain, four chunks, the default (plain)
        if chunks is None:
            os.environ.pop("B200_HCCL_OVERLAP_CHUNKS", None)
        else:
            os.environ["B200_HCCL_OVERLAP_CHUNKS"] = chunks
        o = torch.empty((1100, 512), dtype=torch.float16, device=dev)
        with pkg.use_library(hccl_path):
            pkg.call("aclnnQuantMatmulAllReduce", pkg.AclTensor(bx), pkg.AclTensor(bw), pkg.AclTensor(big["scale"].to(dev)), comm,
                     pkg.AclTensor(o))
        torch.cuda.synchronize()
        outs[chunks] = o
    assert torch.equal(outs["1"], outs["4"]) and torch.equal(outs["1"], outs[None]), f"rank {rank}: chunked all-reduce differs from the plain one"
    acc = oracle.qmm_acc_fast(big["x"].numpy(), big["w"].numpy(), 1100, big["K"], 512)
    assert_close(to_np(outs[None]), oracle.qmm_epilogue_fast(acc, f32(big["scale"])).astype(np.float64), f"rank {rank}: chunked aclnnQuantMatmulAllReduce")
    os.environ["B200_HCCL_OVERLAP_CHUNKS"] = "3"
    dw = workloads.w4a16(M=1030, K=512 * world, N=256, group=128, dtype=torch.float16, per_channel=True, with_bias=False, seed=84)
    kw = slice(rank * 512, (rank + 1) * 512)
    w_r = workloads.pack_int4(dw["w_vals"][kw].contiguous()).to(dev)
    o = torch.empty((1030, 256), dtype=torch.float16, device=dev)
    with pkg.use_library(hccl_path):
        pkg.call("aclnnWeightQuantMatmulAllReduce", pkg.AclTensor(dw["x"][:, kw].contiguous().to(dev)), pkg.AclTensor(w_r, pkg.ACL_INT4, (512, 256)),
                 pkg.AclTensor(dw["scale"].to(dev)), pkg.AclTensor(dw["offset"].to(dev)), comm, pkg.AclTensor(o))
    torch.cuda.synchronize()
    os.environ.pop("B200_HCCL_OVERLAP_CHUNKS", None)
    ref = oracle.wqbmm_fast(f32(dw["x"]), dw["w"].numpy(), True, f32(dw["scale"]), f32(dw["offset"]), None, 1030, dw["K"], 256, 0)
    assert_close(to_np(o), ref, f"rank {rank}: chunked aclnnWeightQuantMatmulAllReduce")

    assert hccl.HcclCommDestroy(comm) == 0
    with open(os.path.join(tmp, f"ok.{rank}"), "w") as f:
        f.write("ok")


if __name__ == "__main__":
    main()
