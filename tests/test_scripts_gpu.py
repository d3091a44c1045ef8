"""Entry points on one GPU: the pre-training script trains in bf16 on the kernel path, evaluates,
writes a checkpoint and resumes from it; both GRPO scripts run two iterations (rollout engine set up
and torn down twice); the diffusion script trains, samples and saves its EMA."""

import os
import re
import subprocess
import sys

import pytest

from tests.helpers import ROOT
from tests.test_scripts_cpu import _corpus

pytestmark = pytest.mark.gpu


def _run(args, env):
    import torch

    if torch.cuda.is_initialized():
        torch.cuda.empty_cache()          # the child sizes its KV pool from the memory that is free now
    full = dict(os.environ, PYTHONPATH=ROOT, **env)
    for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        full.pop(key, None)
    out = subprocess.run([sys.executable] + args, env=full, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    return " ".join((out.stdout + out.stderr).split())


def test_lm_script_on_gpu_trains_checkpoints_and_resumes(tmp_path):
    data, out = str(tmp_path / "data"), str(tmp_path / "out")
    _corpus(data)
    env = {"HB_TEST_DATA": data, "HB_TEST_OUT": out}
    args = [os.path.join(ROOT, "scripts/lm.py"), "--conf", os.path.join(ROOT, "tests/configs/tiny_lm.py"),
            "model.wrapper.param_dtype=bfloat16"]
    logs = _run(args, env)
    losses = [float(x) for x in re.findall(r"global \d+; loss: ([0-9.]+)", logs)]
    assert len(losses) == 4 and losses[-1] < losses[0] - 0.5, logs[-3000:]
    assert "cross entropy" in logs and sorted(os.listdir(out)) == ["step-12", "step-6"]
    logs = _run(args + ["training.max_iter=15"], env)
    assert "resumed at step 12" in logs, logs[-3000:]
    steps = [int(x) for x in re.findall(r"global (\d+); loss", logs)]
    assert steps and min(steps) >= 12


def _prompts(root):
    import json

    from halite_b200.data.sources import RecordFileWriter

    os.makedirs(os.path.join(root, "a"))
    with RecordFileWriter(os.path.join(root, "a", "s0.hbrec")) as w:
        for i in range(64):
            w.write(json.dumps({"text": f"say a lot of a: {i % 7}"}))


@pytest.mark.parametrize("script", ["ppo.py", "ppo_tokainfer.py"])
def test_ppo_scripts_on_gpu(tmp_path, script):
    """GRPO iterations with the in-process engines on the GPU in bf16: rollouts, rewards, updates."""
    data, out = str(tmp_path / "data"), str(tmp_path / "out")
    _prompts(data)
    logs = _run([os.path.join(ROOT, "scripts", script), "--conf", os.path.join(ROOT, "tests/configs/tiny_grpo.py"),
                 "training.max_iter=2", "ppo.actor.parallelize.param_dtype=bfloat16", "ppo.infer_dtype=bfloat16",
                 "ppo.actor.model_conf.dtype=bfloat16", "ppo.inference.memory_fraction=0.15"],
                {"HB_TEST_DATA": data, "HB_TEST_OUT": out})
    steps = [int(x) for x in re.findall(r"global (\d+); actor/", logs)]
    assert steps == [0, 1], logs[-3000:]
    assert "actor/pg_loss" in logs and "critic/rewards_mean" in logs


def test_dit_script_on_gpu(tmp_path):
    out = str(tmp_path / "out")
    logs = _run([os.path.join(ROOT, "scripts/dit.py"), "--conf", os.path.join(ROOT, "tests/configs/tiny_jit.py")],
                {"HB_TEST_OUT": out})
    steps = [int(x) for x in re.findall(r"global (\d+); loss", logs)]
    assert steps == [0, 2, 4, 6, 8], logs[-3000:]
    files = sorted(os.listdir(os.path.join(out, "tiny")))
    assert "ema-0000010.pt" in files and any(f.startswith("samples-0000005") for f in files), files
