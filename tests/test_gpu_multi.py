"""Partitioned chains on real ranks: one process per GPU, halo rows over NCCL (needs two or more GPUs)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_partitioned_chains_over_nccl(built_lib):
    import torch
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(here, "multi_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=os.path.dirname(here))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "multi-GPU parity ok" in r.stdout
