"""Tensor parallelism on CPU / Gloo: sequence-parallel activations, column / row parallel
projections, vocabulary-parallel embedding and cross entropy, combined with sharded data
parallelism; losses and final logits must match a single-process run."""

import os

import pytest

from tests.helpers import ROOT, run_ranks

SCRIPT = os.path.join(ROOT, "tests/ranks/tp_train.py")


@pytest.mark.parametrize("world,tp,split", [(2, 2, "split"), (4, 2, "split"), (2, 2, "fused")])
def test_tensor_parallel_matches_single_process(world, tp, split):
    outs = run_ranks(SCRIPT, world, args=[tp, split], timeout=900)
    assert all("RESULT" in o for o in outs), outs[0][-3000:]
