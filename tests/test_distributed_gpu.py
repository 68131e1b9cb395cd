"""Expert-parallel exchange on 2 (and 4) GPUs of one box: variable-size all-to-all forward
and back, padded variants, locality-aware tail, exchange, and the distributed fabrics.
Runs tests/dist_worker.py under torch.distributed.run; needs at least two GPUs."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("transport", ["p2p", "p2p_small_arena", "p2p_private_copies", "nccl"])
def test_expert_parallel_exchange(world, transport):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", BRT_P2P="0" if transport == "nccl" else "1",
               BRT_P2P_ARENA_MB="1" if transport == "p2p_small_arena" else "64",
               BRT_P2P_ZERO_COPY="0" if transport == "p2p_private_copies" else "1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(HERE / "dist_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert f"DIST_OK {world}" in proc.stdout
