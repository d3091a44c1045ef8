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


@pytest.mark.parametrize("kind", ["adamw", "shampoo"])
def test_plain_optimizer_state_survives_resume(tmp_path, kind):
    """A torch-layout optimizer (lazily built state) saved after a few steps comes back into a
    FRESH optimizer with moments / preconditioner factors / step counts intact, and the next
    update is identical to the uninterrupted run."""
    import torch

    from halite_b200.distributed.checkpoint import CheckpointManager

    def make():
        torch.manual_seed(0)
        model = torch.nn.Linear(16, 8)
        if kind == "adamw":
            opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        else:
            from halite_b200.optim.shampoo import Shampoo

            opt = Shampoo(model.parameters(), lr=1e-2, precondition_frequency=2, start_preconditioning_step=2)
        return model, opt

    def train(model, opt, steps, seed):
        g = torch.Generator().manual_seed(seed)
        for _ in range(steps):
            x = torch.randn(4, 16, generator=g)
            opt.zero_grad()
            model(x).square().mean().backward()
            opt.step()

    model, opt = make()
    train(model, opt, 4, seed=1)
    mgr = CheckpointManager(model, opt, None, directory=str(tmp_path), interval=1)
    assert mgr.save(4, force=True)
    saved = {pid: {k: (v.clone() if torch.is_tensor(v) else v) for k, v in st.items()}
             for pid, st in opt.state_dict()["state"].items()}
    assert saved and all(saved.values())

    model2, opt2 = make()
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(1.0)            # must be overwritten by the load
    mgr2 = CheckpointManager(model2, opt2, None, directory=str(tmp_path), interval=1)
    assert mgr2.load(-1)
    loaded = opt2.state_dict()["state"]
    assert set(loaded) == set(saved)
    for pid, st in saved.items():
        assert set(loaded[pid]) == set(st), (pid, set(loaded[pid]), set(st))
        for name, val in st.items():
            got = loaded[pid][name]
            if torch.is_tensor(val):
                assert torch.equal(got.cpu(), val.cpu()), (pid, name)
            elif isinstance(val, (list, tuple)) and val and torch.is_tensor(val[0]):
                assert all(torch.equal(a, b) for a, b in zip(got, val)), (pid, name)
            else:
                assert got == val, (pid, name)
    train(model, opt, 1, seed=2)
    train(model2, opt2, 1, seed=2)
    for a, b in zip(model.parameters(), model2.parameters()):
        assert torch.equal(a, b)
