"""Sharded data parallelism on CPU / Gloo: the tiny-Llama loss curve and parameters must match a
plain single-process AdamW run (tiny Llama: dim 256, 4 layers, 20 AdamW steps)."""

import os

import pytest

from tests.helpers import ROOT, run_ranks

SCRIPT = os.path.join(ROOT, "tests/ranks/fsdp_train.py")


@pytest.mark.parametrize("mode,world", [("fsdp", 2), ("fsdp", 4), ("hsdp", 4), ("ddp", 2), ("fsdp_micro", 2),
                                        ("ddp_micro", 2), ("ddp_micro_sync", 2), ("fsdp_reshard", 2),
                                        ("fsdp_reshard_micro", 2)])
def test_sharded_training_matches_plain_adamw(mode, world):
    outs = run_ranks(SCRIPT, world, args=[mode], timeout=900)
    assert all("RESULT" in o for o in outs), outs[0][-2000:]
