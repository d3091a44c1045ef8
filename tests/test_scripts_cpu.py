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


def test_lm_script_with_shampoo_on_replicated_ranks(tmp_path):
    """Pre-training with a whole-matrix optimizer: two replicated ranks, Shampoo on fp32 masters of
    the flat buffers, checkpoints written and picked up again."""
    data, out = str(tmp_path / "data"), str(tmp_path / "out")
    _corpus(data)
    env = {"HB_TEST_DATA": data, "HB_TEST_OUT": out}
    script = os.path.join(ROOT, "scripts/lm.py")
    conf = os.path.join(ROOT, "tests/configs/tiny_lm_shampoo.py")
    logs = " ".join(run_ranks(script, 2, args=["--conf", conf], timeout=900, env_extra=env)[0].split())
    losses = [float(x) for x in re.findall(r"global \d+; loss: ([0-9.]+)", logs)]
    assert len(losses) == 4 and losses[-1] < losses[0] - 0.4, logs[-3000:]
    assert sorted(os.listdir(out)) == ["step-12", "step-6"]
    logs = " ".join(run_ranks(script, 2, args=["--conf", conf, "training.max_iter=15"], timeout=900,
                              env_extra=env)[0].split())
    assert "resumed at step 12" in logs, logs[-3000:]


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


def test_eval_task_script_on_a_saved_model_folder(tmp_path, monkeypatch):
    """Save a tiny model folder (config.json + DCP weights + tokenizer config), then run the
    evaluation entry point on a local task; generation is greedy so two runs agree."""
    import sys

    import torch
    import torch.distributed.checkpoint as dcp

    from halite_b200.conf import instantiate, load_config
    from halite_b200.projects.common.config import Model

    section = load_config(os.path.join(ROOT, "tests/configs/tiny_model.py"))
    model_conf = Model(**section)
    torch.manual_seed(0)
    model = instantiate(model_conf.model)
    model.init_weights()
    folder = tmp_path / "model"
    model_conf.save(str(folder))
    dcp.save({"model": model.state_dict()}, checkpoint_id=str(folder))
    assert (folder / "config.json").exists() and (folder / "halite_tokenizer_config.json").exists()

    data = tmp_path / "qa.jsonl"
    with open(data, "w") as f:
        for i in range(6):
            f.write(json.dumps({"problem": f"{i}+{i}", "solution": f"\\boxed{{{2 * i}}}"}) + "\n")
    task = tmp_path / "configs" / "task.py"
    task.parent.mkdir()
    task.write_text(f'''
from halite_b200.conf import field, function
from halite_b200.conf.loader import load_module
from halite_b200.data.preprocess import Map, SelectFeatures
from halite_b200.projects.eval.dataset import jsonl_dataset
_m = load_module("{ROOT}/configs/eval/tasks/minerva_math/eval.py")
conf = field(tasks=[field(
    name="toy_math", dataset=jsonl_dataset("{data}"), evaluate_fn=function(_m.evaluate),
    preprocess=[SelectFeatures(keys=("problem", "solution")), Map(function(_m.record_to_input))],
    sampling_params=field(max_new_tokens=8, top_k=1))])
''')
    sys.path.insert(0, os.path.join(ROOT, "scripts"))
    import eval_task

    monkeypatch.setenv("WORLD_SIZE", "1")
    out = tmp_path / "result.json"
    res = eval_task.main(["--model", str(folder), "--task", str(task), "--device", "cpu", "--output", str(out),
                          "batch_size=4"])
    assert res["toy_math"]["n_samples"] == 6 and 0.0 <= res["toy_math"]["exact_match"] <= 1.0
    assert json.loads(out.read_text())["toy_math"]["n_samples"] == 6


def test_dit_script_trains_samples_and_saves_ema(tmp_path):
    out = str(tmp_path / "out")
    logs = " ".join(run_ranks(os.path.join(ROOT, "scripts/dit.py"), 2,
                              args=["--conf", os.path.join(ROOT, "tests/configs/tiny_jit.py")], timeout=900,
                              env_extra={"HB_TEST_OUT": out})[0].split())
    steps = [int(x) for x in re.findall(r"global (\d+); loss", logs)]
    assert steps == [0, 2, 4, 6, 8], logs[-3000:]
    files = sorted(os.listdir(os.path.join(out, "tiny")))
    assert "ema-0000005.pt" in files and "ema-0000010.pt" in files, files
    assert any(f.startswith("samples-0000005") for f in files)
    import torch

    ema = torch.load(os.path.join(out, "tiny", "ema-0000010.pt"))
    assert "blocks.0.modulator.linear.weight" in ema and ema["head.linear.weight"].shape == (48, 32)


def test_ppo_tokainfer_script_runs(tmp_path):
    data, out = str(tmp_path / "data"), str(tmp_path / "out")
    os.makedirs(os.path.join(data, "a"))
    with RecordFileWriter(os.path.join(data, "a", "s0.hbrec")) as w:
        for i in range(64):
            w.write(json.dumps({"text": f"say a lot of a: {i % 7}"}))
    logs = " ".join(run_ranks(os.path.join(ROOT, "scripts/ppo_tokainfer.py"), 1,
                              args=["--conf", os.path.join(ROOT, "tests/configs/tiny_grpo.py"), "training.max_iter=2"],
                              timeout=900, env_extra={"HB_TEST_DATA": data, "HB_TEST_OUT": out})[0].split())
    steps = [int(x) for x in re.findall(r"global (\d+); actor/", logs)]
    assert steps == [0, 1], logs[-3000:]
    assert "critic/rewards_mean" in logs


def test_ppo_async_script_two_trainers_one_generator(tmp_path):
    data = str(tmp_path / "data")
    os.makedirs(os.path.join(data, "a"))
    with RecordFileWriter(os.path.join(data, "a", "s0.hbrec")) as w:
        for i in range(64):
            w.write(json.dumps({"text": f"say a lot of a: {i % 7}"}))
    outs = run_ranks(os.path.join(ROOT, "scripts/ppo_async.py"), 3,
                     args=["--conf", os.path.join(ROOT, "tests/configs/tiny_grpo.py"), "training.max_iter=3",
                           "monarch.trainer_mesh_size=2", "monarch.generator_mesh_size=1", "output.save_step=100"],
                     timeout=900, env_extra={"HB_TEST_DATA": data, "HB_TEST_OUT": str(tmp_path / "out")})
    logs = " ".join(outs[0].split())
    steps = [int(x) for x in re.findall(r"global (\d+); policy version of rollouts (-?\d+)", logs)
             for x in [x[0]]]
    assert steps == [0, 1, 2], logs[-3000:]
    versions = [int(v) for _, v in re.findall(r"global (\d+); policy version of rollouts (-?\d+)", logs)]
    assert versions[0] == 0 and all(0 <= s - v <= 1 for s, v in zip(steps, versions))
    assert "actor/pg_loss" in logs and "replay buffer dropped" in logs
