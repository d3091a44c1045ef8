"""Tests that need two or more GPUs on one node (skipped otherwise): the fused
compute + collective kernels over real peer memory, and the ctypes NCCL communicator."""

import os
import subprocess
import sys

import pytest
import torch

from tests.helpers import ROOT, free_port, run_ranks

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                 reason="needs at least two GPUs")]


def test_fused_collective_gemms_on_two_gpus():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests/ranks/fused_tp_ranks.py")]
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "RESULT" in out.stdout, (out.stdout + out.stderr)[-3000:]


def test_pynccl_communicator_on_two_gpus():
    outs = run_ranks(os.path.join(ROOT, "tests/ranks/pynccl_ranks.py"), 2, args=[free_port()], timeout=300,
                     env_extra={"HB_TEST_CUDA_VISIBLE": "0,1", "CUDA_VISIBLE_DEVICES": "0,1"})
    assert all("RESULT" in o for o in outs), outs[0][-2000:]


def test_fsdp_parameter_gather_carried_by_gemm_launches():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests/ranks/fsdp_fused_gather_ranks.py")]
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "RESULT ok" in out.stdout, (out.stdout + out.stderr)[-3000:]


def test_tensor_parallel_training_with_collectives_inside_the_gemms():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests/ranks/tp_train_gpu.py")]
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "RESULT ok" in out.stdout, (out.stdout + out.stderr)[-3000:]
