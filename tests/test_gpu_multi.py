"""GPU, two or more devices: the N-sharded GEMMs (NCCL all-gather and one-sided peer stores), row-sharded ops and the
bounded peer wait, one process per GPU (tests/multi_gpu_worker.py).  Skipped on a single GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_gemms_on_two_or_more_gpus():
    world = min(torch.cuda.device_count(), 4)
    port = str(29600 + os.getpid() % 2000)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=port,
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "multi_gpu_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=600)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0] + "\n[timed out]")
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"multi-gpu worker ok rank {r}/{world}" in o, f"rank {r}:\n{o[-3000:]}"
