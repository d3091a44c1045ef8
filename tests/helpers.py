"""Launch helpers for multi-process CPU tests (Gloo ranks on 127.0.0.1)."""

from __future__ import annotations

import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(script: str, world_size: int, args=(), timeout=600, env_extra=None):
    """Run `script` as `world_size` ranks with torchrun-style env; returns rank-0 stdout."""
    port = free_port()
    procs = []
    for rank in range(world_size):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world_size),
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                    "PYTHONPATH": ROOT + os.pathsep + env.get("PYTHONPATH", ""),
                    "CUDA_VISIBLE_DEVICES": env.get("HB_TEST_CUDA_VISIBLE", ""),
                    "OMP_NUM_THREADS": "2"})
        if env_extra:
            env.update(env_extra)
        procs.append(subprocess.Popen([sys.executable, script, *map(str, args)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    failed = None
    for rank, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            failed = failed or (rank, "timeout", out)
        outs.append(out)
        if p.returncode != 0 and failed is None:
            failed = (rank, p.returncode, out)
    if failed is not None:
        raise RuntimeError(f"rank {failed[0]} failed ({failed[1]}):\n{failed[2][-4000:]}")
    return outs
