"""Results of the multi-GPU paths on real peers (needs at least two GPUs; skipped on fewer).

One process per GPU, launched the way the benchmark is; every rank compares what arrived in ITS buffer with
the CPU oracle.  NVLS is switched off and the kernels use plain peer stores, so a rank that fails cannot
disturb the others' GPUs.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_results_match_the_oracle_on_every_rank(world):
    if _gpus() < world:
        pytest.skip(f"UNSUPPORTED: needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="4")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + world), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "MULTI_GPU_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
