"""Sharded matmul on real GPUs over NCCL (needs at least two GPUs in the box; skipped otherwise)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_row_and_batch_shards_gather_to_the_unsharded_product(tv):
    import torch
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("one GPU only")
    worker = Path(__file__).resolve().parent / "multi_gpu_worker.py"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                          "--master-addr", "127.0.0.1", "--master-port", "29577", str(worker)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count(" match=True") == 4
    assert out.stdout.count("fused_match=True") == 4
