"""Time sharding with one process per GPU (CUDA IPC peer memory, plain peer stores, release / acquire flags): needs at
least two GPUs; the single-GPU lock-step form of the same logic is in test_gpu_timeshard.py."""
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,t", [(2, 320), (4, 520)])
def test_time_sharded_processes(cuda, world, t):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = Path(__file__).resolve().parent / "timeshard_worker.py"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(worker), str(t)],
                       capture_output=True, text=True, timeout=600, env=env)
    verdicts = re.findall(r"rank \d+/\d+ T=\d+ samples .*? status \d+ (OK|FAIL)", r.stdout)  # ranks may share a line
    assert r.returncode == 0 and verdicts == ["OK"] * world, r.stdout[-2000:] + r.stderr[-2000:]
