"""Real context parallelism over NCCL: needs at least two GPUs (skipped otherwise).  Spawns torchrun with
tests/cp_worker.py, which compares the sharded NSACore (forward + backward) with the unsharded one on every rank."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_cp_matches_unsharded_over_nccl():
    n = 2 if torch.cuda.device_count() < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(29400 + os.getpid() % 500), os.path.join(HERE, "cp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "CP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
