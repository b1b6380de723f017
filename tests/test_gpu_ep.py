"""Expert-parallel layer on 2 GPUs (NCCL) against the single-GPU layer (outputs within a bf16 rounding step)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expert_parallel_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    worker = Path(__file__).resolve().parent / "ep_worker.py"
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(worker)],
                         capture_output=True, text=True, timeout=600,
                         env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and "EP_CHECK OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
