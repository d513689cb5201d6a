"""Sequence-parallel and sharded forward on two or more GPUs of one node (NCCL send/recv).

Skipped where fewer than two GPUs are visible; the host logic of both paths is covered on CPU by
tests/test_multi_rank_cpu.py.  No TMA multicast is used anywhere in this repository.
"""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sequence_parallel_and_sharded_on_two_gpus():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = min(4, torch.cuda.device_count())
    worker = Path(__file__).with_name("multi_gpu_worker.py")
    with socket.socket() as probe:              # a port that is free right now, instead of a fixed one
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(worker)],
        capture_output=True, text=True, timeout=600)
    lines = [line for line in run.stdout.splitlines() if line.startswith(("OK", "FAIL"))]
    assert run.returncode == 0, run.stderr[-3000:]
    assert len(lines) == world and all(line.startswith("OK") for line in lines), run.stdout[-3000:]
