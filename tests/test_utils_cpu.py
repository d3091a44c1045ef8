"""Training-loop observability helpers: model FLOPs per token, the throughput meter, NVTX phases
(no-ops without a GPU) and the `--profile-steps a:b` window."""

import json
import os
import time
from functools import partial

import pytest
import torch


def _tiny(tie=False):
    from halite_b200.conf import instantiate
    from halite_b200.conf.loader import load_module
    from tests.helpers import ROOT

    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    cfg = zoo.transformer(vocab_size=512, dim=64, n_heads=4, head_dim=16, n_layers=3, intermediate_size=160,
                          context_len=128, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True,
                          gated_ff_split=True, tie_embeds=tie, init=partial(torch.nn.init.normal_, std=0.02))
    return instantiate(cfg)


def test_model_flops_per_token_counts_matmul_parameters_and_attention():
    from halite_b200.utils.throughput import model_flops_per_token

    model = _tiny()
    dim, layers, ff, vocab, S = 64, 3, 160, 512, 128
    qkv = dim * (4 * 16 + 2 * 2 * 16)
    per_layer = qkv + dim * dim + 3 * dim * ff
    matmul = layers * per_layer + vocab * dim            # the head; the embedding lookup is no matmul
    want = 6.0 * matmul + 12.0 * layers * S * dim * 0.5
    got = model_flops_per_token(model, S)
    assert got == pytest.approx(want, rel=1e-6), (got, want)
    # without the causal halving the attention term doubles
    assert model_flops_per_token(model, S, causal=False) - got == pytest.approx(12.0 * layers * S * dim * 0.5)


def test_tied_head_is_counted_once():
    from halite_b200.utils.throughput import model_flops_per_token

    tied, untied = _tiny(tie=True), _tiny(tie=False)
    # the tied matrix does matmul work as the head, so both models do the same FLOPs per token
    assert model_flops_per_token(tied, 64) == pytest.approx(model_flops_per_token(untied, 64), rel=1e-6)


def test_throughput_meter_reports_rates_between_laps(monkeypatch):
    from halite_b200.utils import throughput

    monkeypatch.setenv("HB_PEAK_TFLOPS", "1000")
    clock = {"t": 100.0}
    monkeypatch.setattr(throughput.time, "perf_counter", lambda: clock["t"])
    meter = throughput.ThroughputMeter(flops_per_token=2e9, world_size=8, device="cpu")
    assert meter.lap() == {}                      # first call only sets the mark
    meter.add(4096)
    meter.add(4096)
    clock["t"] += 2.0
    out = meter.lap()
    assert out["tokens_per_s_per_gpu"] == pytest.approx(4096.0)
    assert out["tokens_per_s"] == pytest.approx(8 * 4096.0)
    assert out["tflops_per_gpu"] == pytest.approx(4096.0 * 2e9 / 1e12)
    assert out["mfu"] == pytest.approx(4096.0 * 2e9 / 1e15)
    clock["t"] += 1.0
    assert meter.lap() == {}                      # nothing was added since the last lap


def test_step_window_parsing():
    from halite_b200.utils.nvtx import parse_step_window

    assert parse_step_window(None) is None and parse_step_window("") is None
    assert parse_step_window("3:6") == (3, 6)
    assert parse_step_window("4") == (4, 5)
    with pytest.raises(ValueError):
        parse_step_window("5:5")


def test_step_window_profiler_records_exactly_its_window(tmp_path):
    from halite_b200.utils.nvtx import StepWindowProfiler, phase

    logged = []

    class Log:
        def info(self, msg):
            logged.append(msg)

    prof = StepWindowProfiler((2, 4), output_dir=str(tmp_path), log=Log(), rank=0)
    x = torch.randn(64, 64)
    for step in range(6):
        prof.step_begin(step)
        with phase("forward"):                    # a no-op without a GPU
            x = torch.tanh(x @ x.t() / 64)
        prof.step_end(step)
        assert (prof._prof is not None) == (step in (2,))      # open after step 2 began, closed after step 3
    assert prof.table is not None and "tanh" in prof.table
    assert len(logged) == 1 and "steps 2..3" in logged[0]
    trace = tmp_path / "profile_steps_2_4_rank0.json"
    assert trace.exists()
    events = json.loads(trace.read_text())["traceEvents"]
    assert any("tanh" in str(e.get("name", "")) for e in events)


def test_profile_steps_flag_is_taken_off_the_command_line():
    from halite_b200.conf.loader import load_module
    from halite_b200.utils.nvtx import parse_step_window
    from tests.helpers import ROOT

    pop = load_module(os.path.join(ROOT, "scripts/lm.py")).pop_profile_steps
    argv = ["lm.py", "--conf", "x.py", "--profile-steps", "10:12", "training.max_iter=5"]
    assert parse_step_window(pop(argv)) == (10, 12)
    assert argv == ["lm.py", "--conf", "x.py", "training.max_iter=5"]
    argv = ["lm.py", "--profile-steps=7", "--conf", "x.py"]
    assert parse_step_window(pop(argv)) == (7, 8) and argv == ["lm.py", "--conf", "x.py"]
    assert pop(["lm.py", "--conf", "x.py"]) is None
