"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from halite_b200 import ops

    return ops.ext()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from halite_b200 import ops

    ops.check_status()


def rel_err(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


@pytest.mark.parametrize("layout", ["tn", "nn", "tt", "nt_a_mn"])
@pytest.mark.parametrize("shape", [(128, 128, 64), (512, 768, 1024), (1000, 520, 264), (2048, 1024, 3072), (77, 3072, 4096)])
@pytest.mark.parametrize("bn", [64, 128, 256, 512])   # 512: the CTA-pair kernel (256 x 256 per two SMs)
def test_gemm_layouts(C, layout, shape, bn):
    from halite_b200.ops import gemm

    M, N, K = shape
    a_mn = layout in ("tt", "nt_a_mn")
    b_mn = layout in ("nn", "tt")
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need 16-byte aligned rows")
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=bn)
    ref = A.float() @ B.float().t()
    assert rel_err(out, ref) < 6e-3


def test_gemm_fp32_out_and_accumulate(C):
    from halite_b200.ops import gemm

    torch.manual_seed(1)
    A = torch.randn(1024, 640, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(768, 640, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    out = gemm(A, B, out_dtype=torch.float32)
    assert rel_err(out, ref) < 1e-5
    gemm(A, B, out=out, accumulate=True)
    assert rel_err(out, 2 * ref) < 1e-5
    ob = torch.ones(1024, 768, device="cuda", dtype=torch.bfloat16)
    gemm(A, B, out=ob, accumulate=True)
    assert rel_err(ob, ref + 1) < 6e-3
    # strided output view (columns of a wider buffer)
    wide = torch.zeros(1024, 1024, device="cuda", dtype=torch.bfloat16)
    gemm(A, B, out=wide[:, 128:896])
    assert rel_err(wide[:, 128:896], ref) < 6e-3 and wide[:, :128].abs().max() == 0


@pytest.mark.parametrize("shape", [(5120, 3072, 2048), (640, 256, 8192), (3072, 8192, 1024)])
def test_gemm_split_k_tail_is_exact_and_deterministic(C, shape):
    """Shapes whose last wave is mostly idle take the K-sliced tail schedule: results must match
    the plain schedule's accuracy, accumulate correctly into fp32, and repeat bit for bit."""
    from halite_b200.ops import gemm

    M, N, K = shape
    torch.manual_seed(3)
    A = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)      # wgrad layout: both MN-major
    B = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    ref = A.float().t() @ B.float()
    out = gemm(A, B, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert rel_err(out, ref) < 3e-5
    again = gemm(A, B, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert torch.equal(out, again)
    gemm(A, B, out=out, a_mn=True, b_mn=True, accumulate=True)
    assert rel_err(out, 2 * ref) < 3e-5
    ob = gemm(A, B, a_mn=True, b_mn=True)
    assert rel_err(ob, ref) < 6e-3


@pytest.mark.parametrize("shape", [(5120, 3072, 2048), (4096, 5120, 512), (2560, 8192, 1024), (304, 1000, 4096)])
def test_gemm_pair_kernel_waves_and_split_tail(C, shape):
    """The CTA-pair kernel over several waves of 256 x 256 tiles, with and without a K-sliced last
    wave, in the forward and weight-gradient layouts; results repeat bit for bit."""
    from halite_b200.ops import gemm

    M, N, K = shape
    torch.manual_seed(4)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    out = gemm(A, B, block_n=512)
    assert rel_err(out, ref) < 6e-3
    At, Bt = A.t().contiguous(), B.t().contiguous()
    acc = gemm(At, Bt, a_mn=True, b_mn=True, out_dtype=torch.float32, block_n=512)
    assert rel_err(acc, ref) < 3e-5
    assert torch.equal(acc, gemm(At, Bt, a_mn=True, b_mn=True, out_dtype=torch.float32, block_n=512))
    gemm(At, Bt, out=acc, a_mn=True, b_mn=True, accumulate=True, block_n=512)
    assert rel_err(acc, 2 * ref) < 3e-5
    dgrad = gemm(A, Bt, b_mn=True, block_n=512)
    assert rel_err(dgrad, ref) < 6e-3


@pytest.mark.parametrize("shape", [(64, 2048, 2048), (128, 3072, 3072), (16, 2048, 8192), (100, 1000, 520),
                                   (1, 4096, 1024), (64, 3072, 2048), (8, 1024, 4096), (40, 1280, 1536)])
def test_gemm_cluster_split_k(C, shape):
    """Skinny problems: K split over a cluster of 2 or 4 CTAs, partials summed through distributed
    shared memory. Same accuracy as the plain kernel, bit-identical from launch to launch, both
    output types, accumulate, and the launcher picks it on its own for such shapes."""
    from halite_b200.ops import gemm

    M, N, K = shape
    torch.manual_seed(7)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    out = gemm(A, B, block_n=1064)
    assert rel_err(out, ref) < 6e-3
    assert torch.equal(out, gemm(A, B, block_n=1064))
    assert torch.equal(out, gemm(A, B))                      # block_n = 0 takes the same path
    acc = gemm(A, B, out_dtype=torch.float32, block_n=1064)
    assert rel_err(acc, ref) < 3e-5
    gemm(A, B, out=acc, accumulate=True, block_n=1064)
    assert rel_err(acc, 2 * ref) < 3e-5
    plain = gemm(A, B, out_dtype=torch.float32, block_n=64)
    assert rel_err(acc, 2 * plain) < 3e-5


def test_gemm_pair_kernel_dynamic_schedule_matches_fixed_shares(C):
    """Work items handed out through the counter give the same bits as fixed shares (many waves,
    K-sliced tail included), launch after launch."""
    from halite_b200 import ops
    from halite_b200.ops import gemm

    torch.manual_seed(5)
    A = torch.randn(2048, 5120, device="cuda", dtype=torch.bfloat16)      # [K, M]
    B = torch.randn(2048, 3072, device="cuda", dtype=torch.bfloat16)      # [K, N]: 240 tiles, split tail
    X = torch.randn(8192, 1024, device="cuda", dtype=torch.bfloat16)
    W = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)      # 512 tiles
    ext = ops.ext()
    try:
        ext.gemm_set_dynamic_schedule(False, True)
        fixed = (gemm(A, B, a_mn=True, b_mn=True, out_dtype=torch.float32, block_n=512), gemm(X, W, block_n=512))
        ext.gemm_set_dynamic_schedule(True, True)
        for _ in range(3):
            dyn = (gemm(A, B, a_mn=True, b_mn=True, out_dtype=torch.float32, block_n=512), gemm(X, W, block_n=512))
            assert torch.equal(dyn[0], fixed[0]) and torch.equal(dyn[1], fixed[1])
    finally:
        ext.gemm_set_dynamic_schedule(False, True)
    assert rel_err(fixed[1], X.float() @ W.float().t()) < 6e-3


def test_linear_autograd_matches_torch(C):
    from halite_b200 import ops

    torch.manual_seed(2)
    x = torch.randn(4, 96, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(384, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 1e-2
    assert rel_err(w.grad, wr.grad) < 1e-2
    assert rel_err(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("dim", [256, 1000, 2048, 3072, 4096, 8192])
@pytest.mark.parametrize("residual", [False, True])
def test_rmsnorm(C, dim, residual):
    from halite_b200 import ops
    from halite_b200.ops.norm import rms_norm_reference

    torch.manual_seed(3)
    x = torch.randn(3, 67, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn_like(x).requires_grad_(True) if residual else None
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).bfloat16().requires_grad_(True)
    out = ops.rms_norm(x, w, 1e-5, r)
    y, h = out if residual else (out, None)
    gy = torch.randn_like(y)
    gh = torch.randn_like(y) if residual else None
    if residual:
        torch.autograd.backward([y, h], [gy, gh])
    else:
        y.backward(gy)
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True) if residual else None
    wr = w.detach().float().requires_grad_(True)
    hf = xr + rr if residual else xr
    if residual:
        hf = hf.detach().bfloat16().float() + (hf - hf.detach())   # the kernel rounds the stream to bf16
    yr = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    if residual:
        torch.autograd.backward([yr, hf], [gy.float(), gh.float()])
    else:
        yr.backward(gy.float())
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 2e-2
    assert rel_err(w.grad, wr.grad) < 2e-2
    if residual:
        assert rel_err(r.grad, rr.grad) < 2e-2
        assert rel_err(h, hf) < 1e-2


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_on_slices_of_a_fused_projection(C, interleaved):
    """q and k as strided views of one [tokens, (H + 2 Hk) D] tensor that needs a gradient, with a
    partial rotation (rot_dim < head_dim): the case of every non-packed attention path."""
    from halite_b200 import ops
    from halite_b200.ops.rope import apply_rope_reference, rope_tables

    torch.manual_seed(6)
    T, H, Hk, D, rot = 300, 6, 2, 64, 32
    _rope_on_slices(interleaved, T, H, Hk, D, rot)
    _rope_on_slices(interleaved, 77, 4, 4, 16, 8)        # narrow rotation: the 4-element kernel after a row copy
    # enough tokens for the head-walking form (one thread per token and 8 elements, tables read once
    # per token): partial and full rotation
    _rope_on_slices(interleaved, 16400, 3, 2, 128, 64)
    _rope_on_slices(interleaved, 16400, 2, 1, 128, 128)


def _rope_on_slices(interleaved, T, H, Hk, D, rot):
    from halite_b200 import ops
    from halite_b200.ops.rope import apply_rope_reference, rope_tables

    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2).float() / rot))
    cos, sin = rope_tables(inv, 256, "cuda")
    pos = torch.randint(0, 256, (1, T), device="cuda")
    qkv = torch.randn(1, T, (H + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)

    def run(fn, src):
        q = src[..., : H * D].unflatten(-1, (H, D))
        k = src[..., H * D:(H + Hk) * D].unflatten(-1, (Hk, D))
        v = src[..., (H + Hk) * D:]
        q2, k2 = fn(q, k)
        return (q2.float().square().sum() + (k2.float() * 0.5).sum() + v.float().sum()), q2, k2

    loss, q2, k2 = run(lambda q, k: ops.apply_rope(q, k, cos, sin, pos, interleaved), qkv * 1.0)
    loss.backward()
    ref = qkv.detach().float().requires_grad_(True)
    loss_r, q3, k3 = run(lambda q, k: (apply_rope_reference(q, cos, sin, pos, interleaved),
                                       apply_rope_reference(k, cos, sin, pos, interleaved)), ref)
    loss_r.backward()
    assert rel_err(q2, q3) < 1e-2 and rel_err(k2, k3) < 1e-2
    assert rel_err(qkv.grad, ref.grad) < 2e-2


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_forward_backward(C, interleaved):
    from halite_b200 import ops
    from halite_b200.ops.rope import apply_rope_reference, rope_tables

    torch.manual_seed(4)
    B, S, H, Hk, D = 2, 129, 12, 4, 128
    inv = 1.0 / (500000 ** (torch.arange(0, D, 2).float() / D))
    cos, sin = rope_tables(inv, 512, "cuda")
    pos = torch.randint(0, 512, (B, S), device="cuda")
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hk, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q2, k2 = ops.apply_rope(q.clone(), k.clone(), cos, sin, pos, interleaved)
    gq, gk = torch.randn_like(q2), torch.randn_like(k2)
    torch.autograd.backward([q2, k2], [gq, gk])
    qr = q.detach().float().requires_grad_(True)
    kr = k.detach().float().requires_grad_(True)
    q3 = apply_rope_reference(qr, cos, sin, pos, interleaved)
    k3 = apply_rope_reference(kr, cos, sin, pos, interleaved)
    torch.autograd.backward([q3, k3], [gq.float(), gk.float()])
    assert rel_err(q2, q3) < 1e-2 and rel_err(k2, k3) < 1e-2
    assert rel_err(q.grad, qr.grad) < 1e-2 and rel_err(k.grad, kr.grad) < 1e-2


@pytest.mark.parametrize("kind", ["silu", "gelu_tanh"])
def test_gated_activation(C, kind):
    from halite_b200.ops.activation import gated_act, gated_act_packed

    torch.manual_seed(5)
    p = torch.randn(5, 33, 2 * 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = gated_act_packed(p, kind, gate_first=False)
    g = torch.randn_like(out)
    out.backward(g)
    pr = p.detach().float().requires_grad_(True)
    up, gate = pr[..., :1024], pr[..., 1024:]
    act = torch.nn.functional.silu(gate) if kind == "silu" else torch.nn.functional.gelu(gate, approximate="tanh")
    ref = act * up
    ref.backward(g.float())
    assert rel_err(out, ref) < 1e-2 and rel_err(p.grad, pr.grad) < 2e-2
    a = torch.randn(7, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(7, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    o2 = gated_act(a, b, kind)
    o2.sum().backward()
    assert a.grad is not None and b.grad is not None and o2.shape == a.shape


@pytest.mark.parametrize("vocab", [1000, 32000, 128256])
def test_cross_entropy_rows(C, vocab):
    from halite_b200 import ops
    from halite_b200.ops.loss import cross_entropy_rows_reference

    torch.manual_seed(6)
    R = 65
    logits = (2 * torch.randn(R, vocab, device="cuda")).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, vocab, (R,), device="cuda")
    tgt[3] = -100
    loss, z, lse = ops.cross_entropy_rows(logits, tgt, z_loss=1e-4)
    w = torch.rand(R, device="cuda")
    (loss * w).sum().backward()
    lr = logits.detach().float().requires_grad_(True)
    loss_r, z_r, lse_r = cross_entropy_rows_reference(lr, tgt, z_loss=1e-4)
    (loss_r * w).sum().backward()
    assert torch.allclose(loss, loss_r, atol=2e-3, rtol=1e-4)
    assert torch.allclose(lse, lse_r, atol=1e-3)
    assert torch.allclose(z, z_r, atol=1e-4)
    assert (logits.grad.float() - lr.grad).abs().max() < 2e-2 * lr.grad.abs().max()
    assert logits.grad[3].abs().max() == 0


def test_cross_entropy_softcap_smoothing(C):
    from halite_b200 import ops
    from halite_b200.ops.loss import cross_entropy_rows_reference

    torch.manual_seed(7)
    logits = (3 * torch.randn(33, 5000, device="cuda")).float().requires_grad_(True)
    tgt = torch.randint(0, 5000, (33,), device="cuda")
    loss, _, _ = ops.cross_entropy_rows(logits, tgt, softcap=30.0, label_smoothing=0.1)
    loss.sum().backward()
    lr = logits.detach().clone().requires_grad_(True)
    loss_r, _, _ = cross_entropy_rows_reference(lr, tgt, softcap=30.0, label_smoothing=0.1)
    loss_r.sum().backward()
    assert torch.allclose(loss, loss_r, atol=1e-4, rtol=1e-5)
    assert torch.allclose(logits.grad, lr.grad, atol=1e-5)


def test_fused_linear_cross_entropy(C):
    from halite_b200 import ops

    torch.manual_seed(8)
    T, D, V = 700, 256, 9000
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, D, device="cuda")).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, V, (T,), device="cuda")
    tgt[::7] = -100
    losses, z = ops.fused_linear_cross_entropy(x, w, tgt, z_loss=1e-4, chunk_rows=256)
    losses.mean().backward()
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    logits = xr @ wr.t()
    lse = torch.logsumexp(logits, -1)
    ce = torch.nn.functional.cross_entropy(logits, tgt, reduction="none", ignore_index=-100)
    ref = ce + 1e-4 * lse.square() * (tgt != -100)
    ref.mean().backward()
    assert torch.allclose(losses, ref, atol=3e-2, rtol=1e-2)
    assert rel_err(x.grad, xr.grad) < 3e-2
    assert rel_err(w.grad, wr.grad) < 3e-2


def test_logprob_entropy(C):
    from halite_b200 import ops

    torch.manual_seed(9)
    T, D, V = 300, 128, 5000
    h = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.1 * torch.randn(V, D, device="cuda")).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, V, (T,), device="cuda")
    inv_t = 1.0 / (0.5 + torch.rand(T, device="cuda"))
    logp, ent = ops.logprob_entropy(h, w, tgt, inv_t, chunk_rows=128)
    gl, ge = torch.randn(T, device="cuda"), torch.randn(T, device="cuda")
    torch.autograd.backward([logp, ent], [gl, ge])
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    logits = (hr @ wr.t()).bfloat16().float() * inv_t[:, None]
    lp_all = torch.log_softmax(logits, -1)
    logits2 = (hr @ wr.t()) * inv_t[:, None]
    lp2 = torch.log_softmax(logits2, -1)
    lpr = lp2.gather(-1, tgt[:, None]).squeeze(-1)
    entr = -(lp2.exp() * lp2).sum(-1)
    torch.autograd.backward([lpr, entr], [gl, ge])
    assert torch.allclose(logp, lpr, atol=3e-2)
    assert torch.allclose(ent, entr, atol=3e-2)
    assert rel_err(h.grad, hr.grad) < 4e-2
    assert rel_err(w.grad, wr.grad) < 4e-2


def test_adamw_clip_and_casts(C):
    from halite_b200 import ops

    torch.manual_seed(10)
    n = 100003
    master = torch.randn(n, device="cuda")
    ref = master.clone().requires_grad_(True)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 5):
        g = torch.randn(n, device="cuda")
        ss = torch.zeros(1, device="cuda")
        ops.grad_sumsq(g, ss)
        coef = torch.empty(2, device="cuda")
        C.clip_coef_(ss, 1.0, coef)
        assert abs(coef[1].item() - g.norm().item()) / g.norm().item() < 1e-5
        ref.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref], 1.0)
        opt.step()
        ops.fused_adamw_step(master, m, v, g, low, 1e-2, (0.9, 0.95), 1e-8, 0.1, step, 1.0, coef)
    assert (master - ref.detach()).abs().max() < 1e-5
    assert torch.equal(low, master.bfloat16())
    gb = torch.randn(n, device="cuda").bfloat16()
    ss = torch.zeros(1, device="cuda")
    ops.grad_sumsq(gb, ss)
    assert abs(ss.item() - gb.float().square().sum().item()) / ss.item() < 1e-5


def test_gae(C):
    from halite_b200 import ops
    from halite_b200.ops.rl import gae_reference

    torch.manual_seed(11)
    r, v = torch.randn(17, 93, device="cuda"), torch.randn(17, 93, device="cuda")
    mask = (torch.rand(17, 93, device="cuda") > 0.2).float()
    for m in (None, mask):
        adv, ret = ops.gae(r, v, 0.99, 0.95, m)
        adv_r, ret_r = gae_reference(r, v, 0.99, 0.95, m)
        assert torch.allclose(adv, adv_r, atol=1e-4) and torch.allclose(ret, ret_r, atol=1e-4)


def test_packed_qkv_attention_matches_eager(C):
    from halite_b200.ops.attention import attention_reference, packed_qkv_attention
    from halite_b200.ops.rope import apply_rope_reference, rope_tables

    torch.manual_seed(12)
    B, S, H, Hk, D = 2, 256, 8, 2, 64
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    cos, sin = rope_tables(inv, 512, "cuda")
    pos = torch.arange(S, device="cuda").unsqueeze(0)
    qkv = torch.randn(B, S, (H + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = packed_qkv_attention(qkv.clone(), H, Hk, D, cos, sin, pos, True, True, None)
    g = torch.randn_like(out)
    out.backward(g)
    qr = qkv.detach().float().requires_grad_(True)
    q = qr[..., : H * D].unflatten(-1, (H, D))
    k = qr[..., H * D:(H + Hk) * D].unflatten(-1, (Hk, D))
    v = qr[..., (H + Hk) * D:].unflatten(-1, (Hk, D))
    q = apply_rope_reference(q, cos, sin, pos, True)
    k = apply_rope_reference(k, cos, sin, pos, True)
    ref = attention_reference(q, k, v, causal=True, q_offset=None).reshape(B, S, H * D)
    ref.backward(g.float())
    assert rel_err(out, ref) < 2e-2
    assert rel_err(qkv.grad, qr.grad) < 3e-2


def test_moe_experts_padded_grouped_path_matches_reference(C, monkeypatch):
    """Expert feed-forward on the grouped GEMM modes (device-side tile table, no host sync) against
    the per-expert reference path of the same weights: output and all gradients, with an expert
    that receives no token and with dropped slots."""
    from halite_b200.models.moe.experts import ExpertLinear, FeedForward
    from halite_b200.nn.activation import SwiGLU

    torch.manual_seed(8)
    E, dim, inter, top_k, T = 6, 128, 192, 2, 300
    ff = FeedForward(ExpertLinear(E, dim, 2 * inter), SwiGLU(), ExpertLinear(E, inter, dim), top_k).cuda().bfloat16()
    ff.init_weights()
    with torch.no_grad():
        ff.linear1.weight.mul_(3)
        ff.linear2.weight.mul_(3)
    x = torch.randn(T, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    idx = torch.randint(0, E - 1, (T, top_k), device="cuda")           # expert E-1 never chosen
    idx[::17, 1] = E                                                    # dropped slots
    probs = torch.rand(T, top_k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(T, dim, device="cuda", dtype=torch.bfloat16)

    def run():
        for t in (x, probs, ff.linear1.weight, ff.linear2.weight):
            t.grad = None
        out = ff(x, probs, idx)
        out.backward(g)
        return out.detach().float(), [t.grad.float() for t in (x, probs, ff.linear1.weight, ff.linear2.weight)]

    out, grads = run()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")        # the grouped path must not wait for the device anywhere
    try:
        run()
    finally:
        torch.cuda.set_sync_debug_mode("default")
    monkeypatch.setenv("HALITE_B200_FORCE_REFERENCE", "1")
    out_r, grads_r = run()
    assert rel_err(out, out_r) < 2e-2
    for a, b in zip(grads, grads_r):
        assert rel_err(a, b) < 3e-2
    assert grads[2][E - 1].abs().max() == 0 and grads[3][E - 1].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("reverse", [False, True])
def test_linear_scan_kernel_matches_a_plain_loop(dtype, reverse):
    """h[t] = a[t] h[t-1] + b[t] x[t] per sequence of a packed row: lengths 1, 7, 8, 9 and 275 (the
    kernel fetches eight steps at a time), 200 channels (not a multiple of the CTA width)."""
    from halite_b200.ops.scan import _linear_scan_reference, linear_scan

    torch.manual_seed(0)
    cu = torch.tensor([0, 1, 8, 16, 25, 300], device="cuda", dtype=torch.int32)
    x = torch.randn(300, 200, device="cuda").to(dtype)
    a = torch.rand(300, device="cuda")
    b = torch.rand(300, device="cuda")
    out = linear_scan(x, a, b, cu, reverse=reverse)
    ref = _linear_scan_reference(x.cpu(), a.cpu(), b.cpu(), cu.cpu(), reverse)
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)


def test_ema_scan_gradients_and_dechunk_match_the_chunked_formulation(monkeypatch):
    """`ema_scan` on the GPU against its PyTorch path on CPU (values, dx, dp), then the H-Net dechunk
    with the kernel against the chunked-scan formulation it replaces."""
    from halite_b200.models.models.hnet import dechunk
    from halite_b200.ops.scan import ema_scan

    torch.manual_seed(1)
    cu = torch.tensor([0, 40, 41, 150])
    x = torch.randn(150, 96)
    p = torch.rand(150).clamp(0.05, 0.95)
    w = torch.randn(150, 96)
    got = []
    for dev in ("cpu", "cuda"):
        xd, pd = x.clone().to(dev).requires_grad_(), p.clone().to(dev).requires_grad_()
        out = ema_scan(xd, pd, cu.to(dev))
        (out * w.to(dev)).sum().backward()
        got.append((out.detach().cpu(), xd.grad.cpu(), pd.grad.cpu()))
    for c, g in zip(*got):
        torch.testing.assert_close(g, c, rtol=1e-4, atol=1e-4)

    # dechunk: 3 sequences of 64 tokens, every fourth token (and each first) a boundary
    total = 192
    mask = torch.zeros(total, dtype=torch.bool, device="cuda")
    mask[::4] = True
    prob = torch.rand(total, device="cuda").clamp(0.1, 0.9)
    prob[::64] = 1.0
    bp = torch.stack((1 - prob, prob), -1)
    kept = int(mask.sum())
    cu_kept = torch.tensor([0, 16, 32, 48], device="cuda", dtype=torch.int32)
    inp = torch.randn(1, kept, 64, device="cuda", dtype=torch.bfloat16)
    outs = []
    for force in ("0", "1"):
        monkeypatch.setenv("HALITE_B200_FORCE_REFERENCE", force)
        xi, bi = inp.clone().requires_grad_(), bp.clone().requires_grad_()
        o = dechunk(xi, mask, bi, cu_kept)
        o.float().square().sum().backward()
        outs.append((o.detach().float(), xi.grad.float(), bi.grad[:, 1]))
    assert outs[0][0].shape == (1, total, 64)
    torch.testing.assert_close(outs[0][0], outs[1][0], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(outs[0][1], outs[1][1], rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(outs[0][2], outs[1][2], rtol=5e-2, atol=5e-2)


def test_ssd_scan_state_passing_on_the_recurrence_kernel(monkeypatch):
    """Mamba-2 chunked scan on the GPU: the chunk-to-chunk carry on `linear_scan_kernel` against
    the per-chunk loop (the forced reference path), packed sequences, values and gradients."""
    from halite_b200.models.models.mamba2 import ssd_scan

    b, L, H, P, G, N = 2, 512, 4, 32, 2, 32
    seq = torch.zeros(b, L, dtype=torch.int32, device="cuda")
    seq[:, 200:] = 1
    seq[1, 300:] = 2
    outs = []
    for force in ("1", "0"):
        monkeypatch.setenv("HALITE_B200_FORCE_REFERENCE", force)
        torch.manual_seed(0)
        ins = [torch.randn(b, L, H, P, device="cuda"), torch.rand(b, L, H, device="cuda") * 0.5 + 0.01,
               -torch.rand(H, device="cuda") - 0.1, torch.randn(b, L, G, N, device="cuda"),
               torch.randn(b, L, G, N, device="cuda")]
        ins = [t.requires_grad_() for t in ins]
        y, state = ssd_scan(*ins, chunk_size=64, seq_idx=seq)
        (y.square().mean() + state.square().mean()).backward()
        outs.append([y.detach(), state.detach()] + [t.grad for t in ins])
    for ref, got in zip(*outs):
        torch.testing.assert_close(got, ref, rtol=2e-3, atol=2e-3)
