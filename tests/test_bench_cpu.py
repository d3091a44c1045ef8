"""bench.py command line: presets per model, and the `config` both arms print for one command line."""

import sys

import pytest


def _parse(argv):
    import bench

    old = sys.argv
    sys.argv = ["bench.py", *argv]
    try:
        return bench, bench.parse()
    finally:
        sys.argv = old


def test_headline_defaults_are_the_named_configuration():
    bench, args = _parse([])
    assert (args.gpus, args.metric, args.impl, args.model) == (1, "train", "ours", "llama-3.2-3b")
    assert (args.tp, args.seq_len, args.seqs_per_gpu, args.micro_batches) == (1, 4096, 8, 1)
    assert args.warmup >= 3
    cfg = bench.train_config(args, 8)
    assert cfg["global_batch"] == 64 and cfg["parallelism"] == "fsdp8" and cfg["seq_len"] == 4096


def test_8b_preset_is_tp2_fsdp4_with_global_batch_32():
    bench, args = _parse(["--model", "llama-3-8b", "--gpus", "8"])
    assert (args.tp, args.seq_len, args.seqs_per_gpu, args.micro_batches) == (2, 8192, 8, 2)
    cfg = bench.train_config(args, 8)
    assert cfg == {"model": "llama-3-8b", "global_batch": 32, "seq_len": 8192, "micro_batches": 2,
                   "parallelism": "tp2 x fsdp4",
                   "l2": "inputs larger than L2 (activations of 32768 tokens per pass)"}
    # explicit flags win over the preset (the FSDP-only rows of the same model)
    bench, args = _parse(["--model", "llama-3-8b", "--gpus", "8", "--tp", "1", "--seqs-per-gpu", "4"])
    assert bench.train_config(args, 8)["parallelism"] == "fsdp8" and bench.train_config(args, 8)["global_batch"] == 32


def test_a_debug_layer_count_marks_the_record_invalid():
    bench, args = _parse(["--layers", "2"])
    assert bench.train_config(args, 1)["model"].endswith("INVALID")


def test_both_training_arms_print_the_same_config_object():
    import inspect

    import baseline.reference_bench as ref
    import bench

    assert "train_config(args, world)" in inspect.getsource(ref._run)
    assert "train_config(args, world)" in inspect.getsource(bench.run_ours)


@pytest.mark.parametrize("metric", ["rollout"])
def test_rollout_arms_share_their_config(metric):
    import inspect

    import baseline.reference_rollout as ref
    import bench

    assert "rollout_config" in inspect.getsource(ref) and "rollout_config" in inspect.getsource(bench.run_rollout_ours)
