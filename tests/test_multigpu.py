"""Multi-GPU tests: run tests/dist_worker.py as one process per GPU."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_exchange_and_recovery(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"  # ranks come and go in this test; keep NVLink multicast out of it
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dist_worker.py")
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
        "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker,
    ]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert f"DIST_WORKER_OK {world}" in proc.stdout
