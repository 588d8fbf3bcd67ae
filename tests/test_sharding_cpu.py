"""Multi-rank logic on CPU: two gloo ranks each compute their column shard with the CPU checker,
all-gather the shards and must reproduce the unsharded result (rank-major gather layout, even-column
shard boundaries for packed int4, replicated activations)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, int4, ret):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.load_package()
    from cann_on_gpu_b200 import workloads
    o = ge.load_oracle()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = 3, 256, 192
        full = (workloads.w4a16(M=M, K=K, N=N, group=128, dtype=torch.float32, seed=77) if int4
                else workloads.w8a16(M=M, K=K, N=N, dtype=torch.float32, seed=77, with_offset=True))
        mine = workloads.shard_columns(full, world, rank)
        f = lambda t: None if t is None else t.float().numpy()
        part = o.wqbmm_fast(f(mine["x"]), mine["w"].numpy(), mine["int4"], f(mine["scale"]), f(mine["offset"]), f(mine["bias"]),
                            M, K, mine["N"], mine["group"])
        send = torch.from_numpy(part).contiguous()
        bufs = [torch.empty_like(send) for _ in range(world)]
        dist.all_gather(bufs, send)
        gathered = torch.stack(bufs)                       # [g][M][N/g], what HcclAllGather hands back
        whole = workloads.interleave_gathered(gathered, world, M, N).numpy()
        want = o.wqbmm_fast(f(full["x"]), full["w"].numpy(), full["int4"], f(full["scale"]), f(full["offset"]), f(full["bias"]),
                            M, K, N, full["group"])
        ok = np.allclose(whole, want, rtol=1e-12, atol=1e-12)
        # every rank sees the same activations
        xs = [torch.empty_like(full["x"]) for _ in range(world)]
        dist.all_gather(xs, full["x"].contiguous())
        ok = ok and all(torch.equal(x, xs[0]) for x in xs)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("int4", [False, True])
def test_column_shards_gather_to_the_unsharded_result(int4):
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, port, int4, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_shard_boundaries_keep_nibble_pairs_together():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.load_package()
    from cann_on_gpu_b200 import workloads
    d = workloads.w4a16(M=1, K=64, N=64, group=64, dtype=torch.float32, seed=5)
    parts = [workloads.shard_columns(d, 4, r) for r in range(4)]
    vals = torch.cat([p["w_vals"] for p in parts], dim=1)
    assert torch.equal(vals, d["w_vals"])
    for p in parts:
        assert torch.equal(workloads.pack_int4(p["w_vals"]), p["w"])
    with pytest.raises(AssertionError):
        workloads.shard_columns(d, 64, 0)  # one column per rank would split a byte


FAKE_NCCL = r"""
/* Stand-in for NCCL in the bootstrap test: the unique id is handed out, the rendezvous of more than one rank
   never completes (the other rank never joins), everything else reports success. */
#include <string.h>
#include <unistd.h>
typedef struct { char internal[128]; } ncclUniqueId;
int ncclGetUniqueId(ncclUniqueId *id) { memset(id, 7, sizeof(*id)); return 0; }
int ncclCommInitRank(void **comm, int nranks, ncclUniqueId id, int rank) {
    (void)id; (void)rank;
    if (nranks > 1) for (;;) sleep(1);
    *comm = (void *)0x1;
    return 0;
}
int ncclCommDestroy(void *c) { (void)c; return 0; }
int ncclAllReduce() { return 0; }
int ncclAllGather() { return 0; }
int ncclReduceScatter() { return 0; }
int ncclBroadcast() { return 0; }
int ncclCommCount(void *c, int *n) { (void)c; *n = 1; return 0; }
int ncclCommUserRank(void *c, int *r) { (void)c; *r = 0; return 0; }
"""

BOOTSTRAP_CHILD = r"""
import ctypes, sys, time
hccl = ctypes.CDLL(sys.argv[1])
info = ctypes.create_string_buffer(4108)
assert hccl.HcclGetRootInfo(info) == 0
comm = ctypes.c_void_p()
t0 = time.time()
st = hccl.HcclCommInitRootInfo(ctypes.c_uint32(2), info, ctypes.c_uint32(0), ctypes.byref(comm))   # rank 1 never joins
dt = time.time() - t0
print("status", st, "seconds", round(dt, 2))
assert st == 9 and 0.5 < dt < 10, (st, dt)             # HCCL_E_TIMEOUT, after about the configured second
st = hccl.HcclCommInitRootInfo(ctypes.c_uint32(1), info, ctypes.c_uint32(0), ctypes.byref(comm))   # alone: no rendezvous
assert st == 0 and comm.value
print("ok")
"""


def test_bootstrap_gives_up_on_a_rank_that_never_joins(tmp_path):
    """Failure detection on the host, without a GPU: HcclCommInitRootInfo waits for every rank of the communicator;
    with a peer that never joins it must come back with HCCL_E_TIMEOUT after B200_HCCL_INIT_TIMEOUT_S instead of
    hanging.  NCCL is replaced by a stand-in whose rendezvous never completes (B200_HCCL_NCCL_LIB); the call runs
    in a child process, which takes the abandoned helper thread with it when it exits."""
    import subprocess
    lib_dir = os.path.join(ROOT, "cann-on-gpu_b200", "lib")
    hccl = os.path.join(lib_dir, "libhccl.so")
    if not os.path.exists(hccl):
        pytest.skip("libhccl.so not built (nccl.h absent)")
    src = tmp_path / "fake_nccl.c"
    src.write_text(FAKE_NCCL)
    fake = tmp_path / "libfake_nccl.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", str(fake), str(src)])
    child = tmp_path / "child.py"
    child.write_text(BOOTSTRAP_CHILD)
    env = dict(os.environ, B200_HCCL_NCCL_LIB=str(fake), B200_HCCL_INIT_TIMEOUT_S="1")
    r = subprocess.run([sys.executable, str(child), hccl], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=60)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:]
