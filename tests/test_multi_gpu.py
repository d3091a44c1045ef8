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

# every rank script takes its world size from the launcher: run them on 2 ranks and, where the box
# has them, on 4 (uneven last granules, more than one concurrent peer, tensor x data parallel meshes)
WORLDS = [2, 4]


def _torchrun(script, world, env_extra=None, timeout=600):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, script)]
    env = dict(os.environ, PYTHONPATH=ROOT, **(env_extra or {}))
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("world", WORLDS)
def test_fused_collective_gemms_over_peer_memory(world):
    out = _torchrun("tests/ranks/fused_tp_ranks.py", world)
    assert out.returncode == 0 and "RESULT" in out.stdout, (out.stdout + out.stderr)[-3000:]


def test_pynccl_communicator_on_two_gpus():
    outs = run_ranks(os.path.join(ROOT, "tests/ranks/pynccl_ranks.py"), 2, args=[free_port()], timeout=300,
                     env_extra={"HB_TEST_CUDA_VISIBLE": "0,1", "CUDA_VISIBLE_DEVICES": "0,1"})
    assert all("RESULT" in o for o in outs), outs[0][-2000:]


@pytest.mark.parametrize("world", WORLDS)
def test_fsdp_parameter_gather_carried_by_gemm_launches(world):
    out = _torchrun("tests/ranks/fsdp_fused_gather_ranks.py", world, {"NCCL_NVLS_ENABLE": "0"})
    assert out.returncode == 0 and "RESULT ok" in out.stdout, (out.stdout + out.stderr)[-3000:]


@pytest.mark.parametrize("world", WORLDS)
def test_tensor_parallel_training_with_collectives_inside_the_gemms(world):
    """tp 2 x (world / 2) sharded data-parallel ranks; with 4 ranks the fused GEMMs run beside FSDP collectives."""
    out = _torchrun("tests/ranks/tp_train_gpu.py", world, {"NCCL_NVLS_ENABLE": "0", "NCCL_MAX_CTAS": "16"})
    assert out.returncode == 0 and "RESULT ok" in out.stdout, (out.stdout + out.stderr)[-3000:]
