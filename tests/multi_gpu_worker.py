"""One rank of the two-GPU checks (run by test_multi_gpu.py as `python multi_gpu_worker.py rank world dir`).

Rank r uses GPU r.  The communicator is set up the way an HCCL program does it (tools/mc2_2node.cpp:24-31
of the reference): rank 0 takes HcclGetRootInfo and hands the blob to the others -- here through a file --
then every rank calls HcclCommInitRootInfo.  Checks:
  1. column sharding: each rank multiplies its [K, N/g] shard, HcclAllGather returns [g][M][N/g], the
     interleave is the [M, N] result of the whole problem;
  1b. the same with the gather fused into the matmul's epilogue (peer-memory receive windows), repeated, captured and
      replayed;
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

    # 1b. the same with the gather fused into the matmul's epilogue (aclnnB200WeightQuantMatmulAllGather): the decode
    # kernel stores its rows into the peers' receive windows, a receiver kernel copies them into `gathered`.  Many calls in
    # a row with changing activations (two receive buffers alternate, the call number lives on the device), one to
    # sixteen rows, int4 in both layouts and int8 weights, a row count the decode kernel does not take (plain sequence
    # with HcclAllGather), and a captured graph replayed -- every result against the oracle on the whole layer.
    hccl.HcclB200P2pStatus.restype = ctypes.c_uint32

    def fused_gather(d_full, xdev, gathered_t, packed=None):
        mine_ = workloads.shard_columns(d_full, world, rank)
        key = id(d_full)
        if key not in dev_cache:
            w_ = mine_["w"].to(dev)
            if packed:
                w_ = pkg.pack_weight_nz(w_, d_full["K"], mine_["N"])
            dev_cache[key] = (w_, mine_["scale"].to(dev), None if mine_["offset"] is None else mine_["offset"].to(dev),
                              None if mine_["bias"] is None else mine_["bias"].to(dev))
        w_, sc_, of_, bi_ = dev_cache[key]
        if d_full["int4"]:
            tw_ = (pkg.AclTensor(w_, pkg.ACL_INT4, (d_full["K"], mine_["N"]), fmt=pkg.ACL_FORMAT_FRACTAL_NZ, storage=(w_.numel() * 2,)) if packed
                   else pkg.AclTensor(w_, pkg.ACL_INT4, (d_full["K"], mine_["N"])))
        else:
            tw_ = pkg.AclTensor(w_)
        with pkg.use_library(hccl_path):
            pkg.call("aclnnB200WeightQuantMatmulAllGather", pkg.AclTensor(xdev), tw_, pkg.AclTensor(sc_), None if of_ is None else pkg.AclTensor(of_),
                     None if bi_ is None else pkg.AclTensor(bi_), ctypes.c_int64(d_full["group"]), comm, pkg.AclTensor(gathered_t))
    dev_cache = {}
    gen = torch.Generator().manual_seed(90)
    cases = [(workloads.w4a16(M=1, K=1024, N=512 * world, group=128, dtype=torch.bfloat16, seed=91), False),
             (workloads.w4a16(M=2, K=2048, N=1024 * world, group=128, dtype=torch.float16, seed=92, with_offset=False), True),
             (workloads.w4a16(M=8, K=1024, N=256 * world, group=128, dtype=torch.bfloat16, seed=93, with_bias=False), True),
             (workloads.w4a16(M=16, K=1024, N=512 * world, group=128, dtype=torch.bfloat16, seed=94), False),
             (workloads.w8a16(M=3, K=1024, N=256 * world, dtype=torch.float16, seed=95, with_offset=True), False),
             (workloads.w4a16(M=40, K=1024, N=256 * world, group=128, dtype=torch.bfloat16, seed=96), False)]   # plain sequence
    for ci, (full_c, packed) in enumerate(cases):
        Mc, Nc = full_c["M"], full_c["N"]
        gathered_c = torch.zeros((world, Mc, Nc // world), dtype=full_c["x"].dtype, device=dev)
        for rep in range(3):     # new activations every time, same weights
            xc = torch.randn((Mc, full_c["K"]), generator=gen).to(full_c["x"].dtype)
            gathered_c.fill_(7.0)
            fused_gather(full_c, xc.to(dev), gathered_c, packed)
            torch.cuda.synchronize()
            whole_c = workloads.interleave_gathered(gathered_c, world, Mc, Nc)
            ref_c = oracle.wqbmm_fast(f32(xc), full_c["w"].numpy(), full_c["int4"], f32(full_c["scale"]), f32(full_c["offset"]),
                                      f32(full_c["bias"]), Mc, full_c["K"], Nc, full_c["group"])
            assert_close(to_np(whole_c), ref_c, f"rank {rank}: fused gather, case {ci} call {rep}")
    # captured once, replayed with new activations in the same buffer
    full_g, _ = cases[0]
    xg = torch.zeros((1, full_g["K"]), dtype=torch.bfloat16, device=dev)
    gathered_g = torch.zeros((world, 1, full_g["N"] // world), dtype=torch.bfloat16, device=dev)
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(3):      # three calls per replay: the receive buffers alternate inside a replay and across replays
                fused_gather(full_g, xg, gathered_g, False)
    for rep in range(4):
        xh = torch.randn((1, full_g["K"]), generator=gen).to(torch.bfloat16)
        xg.copy_(xh.to(dev))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        whole_g = workloads.interleave_gathered(gathered_g, world, 1, full_g["N"])
        ref_g = oracle.wqbmm_fast(f32(xh), full_g["w"].numpy(), True, f32(full_g["scale"]), f32(full_g["offset"]), f32(full_g["bias"]),
                                  1, full_g["K"], full_g["N"], 128)
        assert_close(to_np(whole_g), ref_g, f"rank {rank}: fused gather, replay {rep}")
    assert hccl.HcclB200P2pStatus() == 0
    hccl.aclnnB200FusedGatherCount.restype = ctypes.c_uint64
    assert hccl.aclnnB200FusedGatherCount() == 5 * 3 + 3, "the fused form must have run for every case the decode kernel takes"

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
    # decode shapes take the fused form (the kernel sends its partial rows to the peers, a receiver sums them): again with
    # other activations, bf16 int4 weights, one row -- and every rank must end up with the same bits
    hccl.aclnnB200FusedAllReduceCount.restype = ctypes.c_uint64
    assert hccl.aclnnB200FusedAllReduceCount() == 1
    d4 = workloads.w4a16(M=1, K=1024 * world, N=2048, dtype=torch.bfloat16, per_channel=True, with_bias=False, seed=86)
    kq = slice(rank * 1024, (rank + 1) * 1024)
    w4_r = workloads.pack_int4(d4["w_vals"][kq].contiguous()).to(dev)
    for rep in range(3):
        x4 = torch.randn((1, d4["K"]), generator=torch.Generator().manual_seed(870 + rep)).to(torch.bfloat16)
        o4 = torch.empty((1, 2048), dtype=torch.bfloat16, device=dev)
        with pkg.use_library(hccl_path):
            pkg.call("aclnnWeightQuantMatmulAllReduce", pkg.AclTensor(x4[:, kq].contiguous().to(dev)), pkg.AclTensor(w4_r, pkg.ACL_INT4, (1024, 2048)),
                     pkg.AclTensor(d4["scale"].to(dev)), pkg.AclTensor(d4["offset"].to(dev)), comm, pkg.AclTensor(o4))
        torch.cuda.synchronize()
        ref4 = oracle.wqbmm_fast(f32(x4), d4["w"].numpy(), True, f32(d4["scale"]), f32(d4["offset"]), None, 1, d4["K"], 2048, 0)
        assert_close(to_np(o4), ref4, f"rank {rank}: fused all-reduce, call {rep}")
        both = torch.empty((world, 2048), dtype=torch.bfloat16, device=dev)
        assert hccl.HcclAllGather(ctypes.c_void_p(o4.data_ptr()), ctypes.c_void_p(both.data_ptr()), ctypes.c_uint64(2048), ctypes.c_int(HCCL_BF16),
                                  comm, stream) == 0
        torch.cuda.synchronize()
        assert all(torch.equal(both[r], both[0]) for r in range(world)), f"rank {rank}: the ranks' all-reduced results differ"
    assert hccl.aclnnB200FusedAllReduceCount() == 4

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
