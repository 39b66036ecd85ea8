"""Multi-GPU: expert-parallel MegaMoeExperts over peer-mapped buffers, one process per GPU."""

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_oracle(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "_ep_worker.py")]
    result = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout[-6000:] + result.stderr[-1500:]
    assert f"EP={world} ok" in result.stdout
