"""Two-GPU checks of the sharded path: one child process per GPU, NCCL through the Hccl* entry points.
Skipped on a box with fewer than two GPUs (the CPU side of the sharding logic is in
test_sharding_cpu.py)."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_column_shards_gather_and_k_split_allreduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib_dir = os.path.join(os.path.dirname(HERE), "cann-on-gpu_b200", "lib")
    if not os.path.exists(os.path.join(lib_dir, "libhccl.so")):
        pytest.skip("libhccl.so not built")
    world = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with tempfile.TemporaryDirectory() as tmp:
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "multi_gpu_worker.py"), str(r), str(world), tmp],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
        outs = []
        try:
            for p in procs:
                o, _ = p.communicate(timeout=300)
                outs.append(o)
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
        for r, (p, o) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and os.path.exists(os.path.join(tmp, f"ok.{r}")), f"rank {r}:\n{o[-3000:]}"
