"""H-Net and its Mamba-2 mixer on CPU: the chunked scan against the plain recurrence, routing,
chunk / dechunk semantics, causality and sequence isolation of the whole model, a few training
steps from the config file."""

import os

import pytest
import torch
import torch.nn.functional as F

from halite_b200.conf import instantiate, load_config
from halite_b200.models.models.hnet import (Router, chunk, dechunk, get_pos_idx, get_seq_idx, ratio_loss,
                                            straight_through)
from halite_b200.models.models.mamba2 import Mamba2, ssd_scan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _recurrence(x, dt, A, B, C, seq=None):
    b, L, H, P = x.shape
    G, N = B.shape[2:]
    rep = H // G
    y = torch.zeros_like(x)
    for bi in range(b):
        h = torch.zeros(H, P, N)
        for t in range(L):
            if seq is not None and t > 0 and seq[bi, t] != seq[bi, t - 1]:
                h = torch.zeros(H, P, N)
            decay = torch.exp(dt[bi, t] * A)
            Bt, Ct = B[bi, t].repeat_interleave(rep, 0), C[bi, t].repeat_interleave(rep, 0)
            h = h * decay[:, None, None] + dt[bi, t][:, None, None] * x[bi, t][:, :, None] * Bt[:, None, :]
            y[bi, t] = (h * Ct[:, None, :]).sum(-1)
    return y


def test_ssd_scan_matches_recurrence():
    torch.manual_seed(0)
    b, L, H, P, G, N = 2, 75, 4, 8, 2, 6
    x, dt = torch.randn(b, L, H, P), torch.rand(b, L, H) * 0.5 + 0.01
    A = -torch.rand(H) - 0.1
    B, C = torch.randn(b, L, G, N), torch.randn(b, L, G, N)
    seq = torch.zeros(b, L, dtype=torch.long)
    seq[:, 20:] = 1
    seq[:, 51:] = 2            # boundaries both on and off chunk edges (chunk 16)
    seq[:, 64:] = 3
    for s in (None, seq):
        y, _ = ssd_scan(x, dt, A, B, C, chunk_size=16, seq_idx=s)
        torch.testing.assert_close(y, _recurrence(x, dt, A, B, C, s), atol=2e-5, rtol=1e-4)


def test_mamba2_is_causal_and_keeps_packed_sequences_apart():
    torch.manual_seed(0)
    m = Mamba2(32, d_state=16, headdim=16, chunk_size=16)
    m.init_weights()
    u = torch.randn(2, 50, 32)
    out = m(u)
    assert out.shape == u.shape
    changed = u.clone()
    changed[:, 30:] += 1
    torch.testing.assert_close(m(changed)[:, :30], out[:, :30])
    seq = torch.zeros(2, 50, dtype=torch.long)
    seq[:, 21:] = 1
    packed = m(u, seq)
    torch.testing.assert_close(packed[:, 21:], m(u[:, 21:]), atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(packed[:, :21], m(u[:, :21]), atol=1e-5, rtol=1e-4)


def test_index_helpers():
    cu = torch.tensor([0, 3, 3, 7], dtype=torch.int32)
    assert get_seq_idx(cu)[0].tolist() == [0, 0, 0, 2, 2, 2, 2]
    assert get_pos_idx(cu).tolist() == [0, 1, 2, 0, 1, 2, 3]


def test_router_boundaries():
    r = Router(8)
    r.init_weights()
    a, b = torch.randn(8), torch.randn(8)
    x = torch.stack((a, a, -a, -a, b, b))[None]
    out = r(x, cu_seqlens=torch.tensor([0, 4, 6]))
    # identical neighbours: no boundary; opposite neighbours: certain boundary; sequence starts forced
    assert out.boundary_mask.tolist() == [True, False, True, False, True, False]
    torch.testing.assert_close(out.boundary_prob[:, 1], torch.tensor([1.0, 0, 1, 0, 1, 0]), atol=1e-6, rtol=0)
    assert out.selected_prob.shape == (6, 1) and bool((out.selected_prob >= 0.5).all())


def test_chunk_then_dechunk_is_a_per_sequence_ema():
    torch.manual_seed(0)
    total, dim = 12, 4
    x = torch.randn(1, total, dim)
    mask = torch.tensor([1, 0, 1, 1, 0, 0, 1, 0, 0, 1, 1, 0], dtype=torch.bool)
    cu = torch.tensor([0, 6, 12])
    p = torch.rand(total) * 0.8 + 0.1
    prob = torch.stack((1 - p, p), -1)
    kept, next_cu, next_max = chunk(x, mask, cu)
    assert kept.shape == (1, 6, dim) and next_cu.tolist() == [0, 3, 6] and next_max == 3
    out = dechunk(kept, mask, prob, next_cu, n_heads=2, block_size=4)
    expect = torch.zeros(total, dim)
    for s, e in ((0, 6), (6, 12)):
        h = torch.zeros(dim)
        for t in range(s, e):
            if mask[t]:
                h = (1 - p[t]) * h + p[t] * x[0, t]
            expect[t] = h
    torch.testing.assert_close(out[0], expect, atol=1e-5, rtol=1e-4)


def test_ratio_loss_and_straight_through():
    n = 4.0
    mask = torch.tensor([1, 0, 0, 0] * 8, dtype=torch.bool)
    prob = torch.full((32, 2), 0.0)
    prob[:, 1], prob[:, 0] = 1 / n, 1 - 1 / n
    assert abs(float(ratio_loss(n, mask, prob)) - 1.0) < 1e-6
    sure = torch.stack((torch.full((32,), 0.1), torch.full((32,), 0.9)), -1)
    assert float(ratio_loss(n, torch.ones(32, dtype=torch.bool), sure)) > 3.0
    v = torch.tensor([0.3, 0.9], requires_grad=True)
    y = straight_through(v)
    assert y.tolist() == [1.0, 1.0]
    (y * torch.tensor([2.0, 3.0])).sum().backward()
    assert v.grad.tolist() == [2.0, 3.0]


def _tiny():
    torch.manual_seed(0)
    conf = load_config(os.path.join(ROOT, "configs/lm/hnet.py"), "stage2_tiny")
    model = instantiate(conf.model.model)
    model.init_weights("cpu")
    return model


def test_hnet_is_causal_and_rows_do_not_mix():
    model = _tiny().eval()
    ids = torch.randint(0, 256, (3, 48))
    with torch.no_grad():
        base = model(ids)
        later = ids.clone()
        later[:, 30:] = (later[:, 30:] + 7) % 256
        other = ids.clone()
        other[1] = (other[1] + 11) % 256
        out_later, out_other = model(later), model(other)
    assert base.logits.shape == (3, 48, 256)
    assert len(base.router_outputs) == 2 and len(base.aux_outputs) == 2
    torch.testing.assert_close(out_later.logits[:, :30], base.logits[:, :30], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(out_other.logits[[0, 2]], base.logits[[0, 2]], atol=1e-5, rtol=1e-4)
    # each stage shortens the row, and every sequence keeps its first token
    kept = [int(r.boundary_mask.sum()) for r in base.router_outputs]
    assert 3 <= kept[1] <= kept[0] <= 3 * 48


def test_hnet_trains_from_config():
    model = _tiny()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    pattern = torch.arange(48) % 7
    ids = torch.stack([(pattern + k) % 256 for k in range(4)])
    losses = []
    for _ in range(30):
        out = model(ids[:, :-1])
        loss = F.cross_entropy(out.logits.flatten(0, 1).float(), ids[:, 1:].flatten())
        total = loss + sum(a["ratio_loss"] for a in out.aux_outputs)
        opt.zero_grad()
        total.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert all(p.grad is not None for p in model.parameters())
    assert losses[-1] < 0.5 * losses[0], losses


def test_hnet_through_sharded_optimisation_step():
    """The whole model as one flat-buffer unit, the ratio losses picked up from `aux_outputs`."""
    from functools import partial

    from halite_b200.nn.loss import CrossEntropyLoss
    from halite_b200.optim import build_optimizer
    from halite_b200.parallel import parallelize
    from halite_b200.projects.common.train_fn import optimization_step

    torch.manual_seed(0)
    conf = load_config(os.path.join(ROOT, "configs/lm/hnet.py"), "stage2_tiny")
    model = parallelize(instantiate(conf.model.model), param_dtype="float32", reduce_dtype="float32")
    model.init_weights("cpu")
    opt = build_optimizer(partial(torch.optim.AdamW, lr=3e-3), model, weight_decay=0.0)
    pattern = torch.arange(48) % 7
    ids = torch.stack([(pattern + k) % 256 for k in range(4)])
    first = last = None
    for _ in range(16):
        res = optimization_step(model, {"input": ids[:, :-1], "target": ids[:, 1:]}, opt,
                                criterion=CrossEntropyLoss(), clip_grad_norm=1.0)
        last = float(res["loss_dict"]["cross entropy"])
        first = last if first is None else first
        assert "ratio_loss" in res["loss_dict"]
    assert last < 0.5 * first


def test_ema_scan_matches_a_plain_loop_with_gradients():
    """The recurrence front-end (CPU path of `ops/scan.py`) against a naive float64 loop: values and
    both gradients, over sequences of length 4, 1 and 6 in one packed row."""
    from halite_b200.ops.scan import ema_scan

    torch.manual_seed(0)
    total, dim = 11, 5
    cu = torch.tensor([0, 4, 5, 11])
    x = torch.randn(total, dim, dtype=torch.float64, requires_grad=True)
    p = torch.rand(total, dtype=torch.float64).clamp(0.05, 0.95).requires_grad_()
    w = torch.randn(total, dim, dtype=torch.float64)
    rows = []
    for lo, hi in zip(cu.tolist()[:-1], cu.tolist()[1:]):
        h = torch.zeros(dim, dtype=torch.float64)
        for t in range(lo, hi):
            h = (1 - p[t]) * h + p[t] * x[t]
            rows.append(h)
    ref = torch.stack(rows)
    (ref * w).sum().backward()
    xf, pf = x.detach().float().requires_grad_(), p.detach().float().requires_grad_()
    out = ema_scan(xf, pf, cu)
    (out * w.float()).sum().backward()
    torch.testing.assert_close(out, ref.float(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(xf.grad, x.grad.float(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(pf.grad, p.grad.float(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("packed", [False, True])
def test_ssd_scan_state_passing_by_recurrence_matches_the_chunk_loop(monkeypatch, packed):
    """The chunk-to-chunk carry of `ssd_scan` as one linear recurrence over the chunk axis (the GPU
    form, here on the PyTorch path of the scan op) against the per-chunk loop: output, final state
    and every gradient."""
    import halite_b200.models.models.mamba2 as m

    b, L, H, P, G, N = 2, 192, 4, 8, 2, 16
    seq = None
    if packed:
        seq = torch.zeros(b, L, dtype=torch.int32)
        seq[:, 70:] = 1
        seq[:, 130:] = 2
        seq[1, 150:] = 3

    def run(use_scan):
        monkeypatch.setattr(m, "_scan_kernel_for", lambda x: use_scan)
        torch.manual_seed(0)
        ins = [torch.randn(b, L, H, P), torch.rand(b, L, H) * 0.5 + 0.01, -torch.rand(H) - 0.1,
               torch.randn(b, L, G, N), torch.randn(b, L, G, N)]
        ins = [t.requires_grad_() for t in ins]
        y, state = m.ssd_scan(*ins, chunk_size=64, seq_idx=seq)
        (y.square().sum() + state.square().sum()).backward()
        return [y.detach(), state.detach()] + [t.grad for t in ins]

    loop, scan = run(False), run(True)
    assert loop[1].abs().max() > 0
    for a, c in zip(loop, scan):
        torch.testing.assert_close(c, a, rtol=1e-5, atol=1e-5)
