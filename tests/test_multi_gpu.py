"""Multi-GPU checks that need more than one device: run only where at least two GPUs are visible.

The N-rank paths are also covered on one GPU with the ranks emulated (tests/test_embedding_gpu.py) and on
CPU with gloo (tests/test_sharding_cpu.py); this file runs the real thing: one process per GPU, peer-mapped
memory, the library's own barrier between the ranks."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_peer_exchange_matches_the_single_rank_gradient(ranks):
    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs, {torch.cuda.device_count()} visible")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + ranks),
           str(ROOT / "tests" / "peer_exchange_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    for r in range(ranks):
        assert f"PEER_EXCHANGE_OK {r}" in res.stdout
