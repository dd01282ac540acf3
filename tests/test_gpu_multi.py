"""Runs the tensor-parallel parity check on 2 GPUs when the box has them (skipped on one GPU)."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_tensor_parallel_layers_match_oracle():
    import socket

    script = Path(__file__).parent / "multi_gpu_check.py"
    with socket.socket() as sock:  # a free port: the machine is shared
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", str(port), str(script)],
        capture_output=True, text=True, timeout=1200, env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "multi_gpu_check: OK" in res.stdout
