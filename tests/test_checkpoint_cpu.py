"""Checkpoint manager over Gloo ranks: interval saves, pruning, exact resume, async writes and
resuming on a different number of ranks (reference behaviour: distributed/checkpoint.py:78-388)."""

import os

import pytest

from tests.helpers import ROOT, run_ranks

SCRIPT = os.path.join(ROOT, "tests/ranks/ckpt_train.py")


@pytest.mark.parametrize("phase", ["save", "save_async"])
def test_save_resume_and_reshard(tmp_path, phase):
    d = str(tmp_path / "ckpt")
    outs = run_ranks(SCRIPT, 2, args=[d, phase], timeout=600)
    assert all("replay_diff" in o for o in outs), outs[0][-2000:]
    if phase == "save":
        outs = run_ranks(SCRIPT, 4, args=[d, "resume"], timeout=600)
        assert all("reshard_diff" in o for o in outs), outs[0][-2000:]
        # three ranks pad the flat buffers differently: exercises the whole-entry fallback
        outs = run_ranks(SCRIPT, 3, args=[d, "resume"], timeout=600)
        assert all("reshard_diff" in o for o in outs), outs[0][-2000:]
