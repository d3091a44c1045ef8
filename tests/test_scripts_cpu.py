"""Entry points end to end on CPU: `scripts/lm.py` trains the tiny model over two Gloo ranks from
a record-file corpus, evaluates, checkpoints, and a second launch resumes where the first
stopped."""

import json
import os
import re

from halite_b200.data.sources import RecordFileWriter
from tests.helpers import ROOT, run_ranks


def _corpus(root):
    for name, n in (("a", 200), ("b", 50)):
        os.makedirs(os.path.join(root, name))
        with RecordFileWriter(os.path.join(root, name, "s0.hbrec")) as w:
            for i in range(n):
                w.write(json.dumps({"text": f"{name} sample {i}: " + "the quick brown fox " * (1 + i % 3)}))


def test_lm_script_trains_checkpoints_and_resumes(tmp_path):
    data, out = str(tmp_path / "data"), str(tmp_path / "out")
    _corpus(data)
    env = {"HB_TEST_DATA": data, "HB_TEST_OUT": out}
    script = os.path.join(ROOT, "scripts/lm.py")
    conf = os.path.join(ROOT, "tests/configs/tiny_lm.py")
    logs = " ".join(run_ranks(script, 2, args=["--conf", conf], timeout=900, env_extra=env)[0].split())
    losses = [float(x) for x in re.findall(r"global \d+; loss: ([0-9.]+)", logs)]
    assert len(losses) == 4 and losses[-1] < losses[0] - 0.5, logs[-3000:]
    assert "cross entropy" in logs and "loss/a" in logs
    assert sorted(os.listdir(out)) == ["step-12", "step-6"]
    assert os.path.exists(os.path.join(out, "step-12", "config.json"))
    # second launch with a larger budget picks up at step 12
    logs = " ".join(run_ranks(script, 2, args=["--conf", conf, "training.max_iter=15"], timeout=900,
                              env_extra=env)[0].split())
    assert "resumed at step 12" in logs, logs[-3000:]
    steps = [int(x) for x in re.findall(r"global (\d+); loss", logs)]
    assert steps and min(steps) >= 12


def test_ppo_script_runs_grpo_iterations_and_checkpoints(tmp_path):
    data, out = str(tmp_path / "data"), str(tmp_path / "out")
    os.makedirs(os.path.join(data, "a"))
    with RecordFileWriter(os.path.join(data, "a", "s0.hbrec")) as w:
        for i in range(64):
            w.write(json.dumps({"text": f"say a lot of a: {i % 7}"}))
    env = {"HB_TEST_DATA": data, "HB_TEST_OUT": out}
    script = os.path.join(ROOT, "scripts/ppo.py")
    conf = os.path.join(ROOT, "tests/configs/tiny_grpo.py")
    logs = " ".join(run_ranks(script, 2, args=["--conf", conf], timeout=900, env_extra=env)[0].split())
    assert "ppo epochs: 1, minibatches: 1, microbatches: 2" in logs, logs[-3000:]
    steps = [int(x) for x in re.findall(r"global (\d+); actor/", logs)]
    assert steps == [0, 1, 2, 3], logs[-3000:]
    assert "actor/pg_loss" in logs and "critic/rewards_mean" in logs and "sample/response_len/mean" in logs
    assert "[reward]" in logs and "[output]" in logs
    assert sorted(os.listdir(out)) == ["step-2", "step-4"]
