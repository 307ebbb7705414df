"""Host-side distributed logic on CPU ranks (gloo)."""

import os
import socket
import subprocess
import sys


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_cpu_ranks_agree_on_shares():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpu_dist_worker.py")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
        "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker,
    ]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "CPU_DIST_OK 2" in proc.stdout
