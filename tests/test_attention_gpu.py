"""The tcgen05 training attention kernels (forward and backward) against eager fp32 attention
on the same bf16 inputs: causal / full, grouped-query heads, head_dim 64 and 128, sequence
lengths that are not multiples of the tile, sliding windows, soft-capping, packed sequences
(`cu_seqlens`), per-row document offsets and document ids, and the packed-QKV + RoPE path."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, **kw):
    from halite_b200.ops.attention import attention_reference

    return attention_reference(q.float(), k.float(), v.float(), q_offset=None, **kw)


def _check(out, ref, what, tol=2.5e-2):
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * max(scale, 1.0), f"{what}: max err {err:.4f} (ref max {scale:.3f})"


def _run(B, S, Hq, Hk, D, seed=0, grads=True, ref_kw=None, **kw):
    import halite_b200.ops as ops
    from halite_b200.ops.attention import attention

    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(B, S, h, D, device="cuda", generator=g).bfloat16().requires_grad_(grads)
               for h in (Hq, Hk, Hk))
    out = attention(q, k, v, **kw)
    ops.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_(grads) for t in (q, k, v))
    ref = _ref(qr, kr, vr, **(ref_kw if ref_kw is not None else kw))
    _check(out, ref, "out")
    if grads:
        go = torch.randn(out.shape, device="cuda", generator=g).bfloat16()
        out.backward(go)
        ops.check_status()
        ref.backward(go.float())
        for name, a, b in (("dq", q, qr), ("dk", k, kr), ("dv", v, vr)):
            _check(a.grad, b.grad, name)
    return out


@pytest.mark.parametrize("B,S,Hq,Hk,D", [(2, 512, 6, 2, 128), (1, 384, 4, 4, 64), (2, 200, 8, 2, 128),
                                         (1, 1000, 3, 1, 64), (1, 130, 2, 2, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_dense_batches(B, S, Hq, Hk, D, causal):
    _run(B, S, Hq, Hk, D, causal=causal)


def test_llama_head_layout_long_sequence():
    # 24 query / 8 key-value heads as in the 3B model, several key tiles per query tile
    _run(1, 2048, 24, 8, 128, causal=True, grads=True)


@pytest.mark.parametrize("window", [1, 100, 128, 300])
def test_sliding_window(window):
    _run(2, 640, 4, 2, 128, causal=True, window=window)
    _run(1, 333, 4, 4, 64, causal=False, window=window)


@pytest.mark.parametrize("D", [64, 128])
def test_softcap(D):
    _run(2, 300, 4, 2, D, causal=True, softcap=20.0)
    _run(1, 256, 2, 2, D, causal=True, softcap=5.0, window=77)


def _packed_reference(q, k, v, bounds, **kw):
    outs = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e > s:
            outs.append(_ref(q[:, s:e], k[:, s:e], v[:, s:e], **kw))
    return torch.cat(outs, 1)


@pytest.mark.parametrize("lengths", [[37, 300, 129, 1, 513], [128, 128, 256], [700], [5, 5, 5, 5, 1000]])
@pytest.mark.parametrize("causal", [True, False])
def test_packed_sequences_with_cu_seqlens(lengths, causal):
    import halite_b200.ops as ops
    from halite_b200.ops.attention import attention

    total = sum(lengths)
    bounds = [0]
    for n in lengths:
        bounds.append(bounds[-1] + n)
    cu = torch.tensor(bounds, device="cuda", dtype=torch.int32)
    g = torch.Generator(device="cuda").manual_seed(3)
    Hq, Hk, D = 6, 2, 128
    q, k, v = (torch.randn(1, total, h, D, device="cuda", generator=g).bfloat16().requires_grad_() for h in (Hq, Hk, Hk))
    with torch.cuda.device(0):
        torch.cuda.set_sync_debug_mode("error")      # the packed path must not read lengths back
        try:
            out = attention(q, k, v, causal=causal, cu_seqlens=cu)
            go = torch.randn(out.shape, device="cuda", generator=g).bfloat16()
            out.backward(go)
        finally:
            torch.cuda.set_sync_debug_mode("default")
    ops.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _packed_reference(qr, kr, vr, bounds, causal=causal)
    ref.backward(go.float())
    _check(out, ref, "out")
    for name, a, b in (("dq", q, qr), ("dk", k, kr), ("dv", v, vr)):
        _check(a.grad, b.grad, name)


def test_document_offsets_and_ids_inside_rows():
    from halite_b200.models.flex_attention import batch_length_to_offsets
    from halite_b200.ops.attention import attention

    B, S, Hq, Hk, D = 2, 512, 4, 2, 128
    lengths = [[100, 29, 383], [255, 257]]       # boundaries inside tiles and on a tile edge + 1
    offsets = batch_length_to_offsets(lengths, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn(B, S, h, D, device="cuda", generator=g).bfloat16().requires_grad_() for h in (Hq, Hk, Hk))
    out = attention(q, k, v, causal=True, document_offsets=offsets)
    go = torch.randn(out.shape, device="cuda", generator=g).bfloat16()
    out.backward(go)
    ids = torch.zeros(B, S, dtype=torch.long, device="cuda")
    for b, row in enumerate(lengths):
        at = 0
        for d, n in enumerate(row):
            ids[b, at:at + n] = d
            at += n
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref(qr, kr, vr, causal=True, document_ids=ids)
    ref.backward(go.float())
    _check(out, ref, "out")
    for name, a, b in (("dq", q, qr), ("dk", k, kr), ("dv", v, vr)):
        _check(a.grad, b.grad, name)
    out2 = attention(q.detach(), k.detach(), v.detach(), causal=True, document_ids=ids)
    assert torch.equal(out2, out.detach())


@pytest.mark.parametrize("Hq,Hk,D", [(24, 8, 128), (4, 4, 64)])
def test_packed_qkv_with_rope_matches_separate_tensors(Hq, Hk, D):
    import halite_b200.ops as ops
    from halite_b200.ops.attention import packed_qkv_attention
    from halite_b200.ops.rope import apply_rope_reference, rope_tables

    B, S = 2, 384
    g = torch.Generator(device="cuda").manual_seed(7)
    qkv = torch.randn(B, S, (Hq + 2 * Hk) * D, device="cuda", generator=g).bfloat16()
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    cos, sin = rope_tables(inv_freq, S, device="cuda")
    pos = torch.arange(S, device="cuda").unsqueeze(0)
    x = qkv.clone().requires_grad_()
    out = packed_qkv_attention(x * 1, Hq, Hk, D, cos, sin, pos, True, True, None)
    go = torch.randn(out.shape, device="cuda", generator=g).bfloat16()
    out.backward(go)
    ops.check_status()
    xr = qkv.float().requires_grad_()
    qd, kd = Hq * D, Hk * D
    q = apply_rope_reference(xr[..., :qd].unflatten(-1, (Hq, D)), cos, sin, pos, True)
    k = apply_rope_reference(xr[..., qd:qd + kd].unflatten(-1, (Hk, D)), cos, sin, pos, True)
    v = xr[..., qd + kd:].unflatten(-1, (Hk, D))
    ref = _ref(q, k, v, causal=True).reshape(B, S, qd)
    ref.backward(go.float())
    _check(out, ref, "out")
    _check(x.grad, xr.grad, "dqkv")


def test_runs_are_bit_identical_forward():
    from halite_b200.ops.attention import attention

    g = torch.Generator(device="cuda").manual_seed(11)
    q, k, v = (torch.randn(2, 768, h, 128, device="cuda", generator=g).bfloat16() for h in (6, 2, 2))
    a = attention(q, k, v, causal=True)
    b = attention(q, k, v, causal=True)
    assert torch.equal(a, b)
