"""Fused compute + collective GEMM variants on one GPU: the peers' buffers are stand-in local
tensors and their flags are pre-set, so copy CTAs, flag-gated tiles, the scatter epilogue and
the in-kernel reduction all run inside a single launch. The two-GPU path is exercised by
tests/ranks/fused_tp_ranks.py."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _i32(n, val=0):
    return torch.full((n,), val, dtype=torch.int32, device="cuda")


@pytest.fixture
def sm_margin():
    """Leave 20 SMs free in the launches that spin on a peer, as tensor parallelism beside
    data-parallel collectives does."""
    from halite_b200 import ops

    ops.ext().gemm_set_peer_wait_sm_margin(20)
    yield 20
    ops.ext().gemm_set_peer_wait_sm_margin(0)


@pytest.mark.parametrize("rank", [0, 1, 2])
def test_allgather_gemm_a_operand(rank):
    _allgather_gemm_a_operand(rank, 3, 256, 1024, 1536)


def test_fused_modes_keep_working_with_an_sm_margin(sm_margin):
    from halite_b200 import ops

    assert ops.ext().gemm_peer_wait_sm_margin() == 20
    _allgather_gemm_a_operand(1, 2, 2048, 1024, 4096)       # 512 tiles on 128 - 8 compute CTAs
    _gemm_reduce_scatter(0, 2, 2048, 512, 4096)


def _allgather_gemm_a_operand(rank, world, rows, K, N):
    from halite_b200 import ops
    from halite_b200.ops import gemm

    torch.manual_seed(0)
    shards = [torch.randn(rows, K, device="cuda").bfloat16() for _ in range(world)]
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    staging = torch.zeros(world * rows, K, device="cuda", dtype=torch.bfloat16)
    staging[rank * rows:(rank + 1) * rows] = shards[rank]
    epoch = 7
    ready, done = _i32(world, epoch), _i32(world)
    flags = _i32(world * rows // 128)
    counter = _i32(1)
    gather = dict(
        src_ptrs=[0 if c == rank else shards[c].data_ptr() for c in range(world)],
        peer_done_ptrs=[0 if c == rank else done[c:].data_ptr() for c in range(world)],
        dst_ptr=staging.data_ptr(), chunk_bytes=rows * K * 2, granule_bytes=128 * K * 2, n_copy_ctas=8,
        flags_ptr=flags.data_ptr(), ready_ptr=ready.data_ptr(), done_counter_ptr=counter.data_ptr(),
        epoch=epoch, dep=1, dep_row_bytes=K * 2, dep_base_offset=0, m_rot=rank * rows // 128,
        first_chunk=rank)
    y = gemm(staging, w, gather=gather)
    torch.cuda.synchronize()
    ops.check_status()
    full = torch.cat(shards, 0)
    assert torch.equal(staging, full)
    ref = full.float() @ w.float().t()
    assert ((y.float() - ref).abs().max() / ref.abs().max()) < 6e-3
    assert (flags == epoch).all()
    want_done = [0 if c == rank else epoch for c in range(world)]
    assert done.tolist() == want_done


def test_allgather_gemm_b_operand_inside_flat_buffer():
    """FSDP case: the weight of the GEMM is a slice of a flat parameter buffer whose remote
    shards arrive during the launch."""
    from halite_b200 import ops
    from halite_b200.ops import gemm

    torch.manual_seed(1)
    world, rank = 4, 1
    N, K, M = 1024, 512, 640
    pad_front = 4096                      # another parameter sits before the weight in the unit
    total = pad_front + N * K + 8192
    chunk = (total + world - 1) // world
    chunk = (chunk + 127) // 128 * 128
    flat_full = torch.randn(world * chunk, device="cuda").bfloat16()
    flat = torch.zeros_like(flat_full)
    flat[rank * chunk:(rank + 1) * chunk] = flat_full[rank * chunk:(rank + 1) * chunk]
    peers = [flat_full[c * chunk:(c + 1) * chunk].clone() for c in range(world)]
    x = torch.randn(M, K, device="cuda").bfloat16()
    weight = flat[pad_front:pad_front + N * K].view(N, K)
    epoch = 3
    gran = 64 * 1024
    n_gran = world * ((chunk * 2 + gran - 1) // gran)
    flags, ready, counter = _i32(n_gran), _i32(world, epoch), _i32(1)
    gather = dict(
        src_ptrs=[0 if c == rank else peers[c].data_ptr() for c in range(world)],
        dst_ptr=flat.data_ptr(), chunk_bytes=chunk * 2, granule_bytes=gran, n_copy_ctas=4,
        flags_ptr=flags.data_ptr(), ready_ptr=ready.data_ptr(), done_counter_ptr=counter.data_ptr(),
        epoch=epoch, dep=2, dep_row_bytes=K * 2, dep_base_offset=pad_front * 2, first_chunk=rank)
    y = gemm(x, weight, gather=gather)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(flat, flat_full)
    ref = x.float() @ flat_full[pad_front:pad_front + N * K].view(N, K).float().t()
    assert ((y.float() - ref).abs().max() / ref.abs().max()) < 6e-3


@pytest.mark.parametrize("gemm_shape", [(512, 384, 256), (4096, 5120, 512)])
def test_reduce_scatter_slice_carried_by_a_gemm_launch(gemm_shape):
    """Reduce mode of the copy CTAs, four ranks' fp32 buffers emulated in local memory: the
    launch computes its GEMM and, beside it, scale * (sum of the ranks' slices) in rank order.
    The small GEMM runs on the single-CTA kernel, the large one on the CTA-pair kernel (whose
    first clusters then do the reduction)."""
    from halite_b200 import ops
    from halite_b200.ops import gemm

    torch.manual_seed(3)
    world, rank, n = 4, 2, 1 << 20
    grads = [torch.randn(world * n, device="cuda") for _ in range(world)]      # every rank's full buffer
    out = torch.zeros(n, device="cuda")
    epoch = 7
    ready, done, counter = _i32(world, epoch), _i32(world), _i32(1)
    M, N, K = gemm_shape
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    gather = dict(
        src_ptrs=[g[rank * n:].data_ptr() for g in grads], dst_ptr=0, chunk_bytes=16, granule_bytes=16,
        n_copy_ctas=8, flags_ptr=0, ready_ptr=ready.data_ptr(), done_counter_ptr=counter.data_ptr(),
        peer_done_ptrs=[0 if c == rank else done[c:].data_ptr() for c in range(world)],
        epoch=epoch, dep=0, dep_row_bytes=0, first_chunk=rank,
        reduce_out_ptr=out.data_ptr(), reduce_numel=n, reduce_scale=0.25)
    y = gemm(x, w, gather=gather)
    torch.cuda.synchronize()
    ops.check_status()
    want = grads[0][rank * n:(rank + 1) * n].clone()
    for g in grads[1:]:
        want += g[rank * n:(rank + 1) * n]
    assert torch.equal(out, want * 0.25)
    assert done.tolist() == [epoch if c != rank else 0 for c in range(world)]
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).abs().max() / ref.abs().max()) < 6e-3


@pytest.mark.parametrize("rank", [0, 1])
def test_gemm_reduce_scatter(rank):
    _gemm_reduce_scatter(rank, 2, 384, 768, 1024)


def _gemm_reduce_scatter(rank, world, rows, K, N):
    from halite_b200 import ops
    from halite_b200.ops import gemm

    torch.manual_seed(2)
    x = torch.randn(world * rows, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    partial = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    peer_mem = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)      # stands for the peer's receive slot
    from_peer = torch.randn(rows, N, device="cuda").bfloat16()                # what the peer pushed to us
    out = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    epoch = 5
    my_flags, peer_flags, counter = _i32(world, epoch), _i32(world), _i32(1)
    other = 1 - rank
    scatter = dict(
        dst_ptrs=[partial.data_ptr() if c == rank else peer_mem.data_ptr() for c in range(world)],
        recv_ptrs=[0 if p == rank else from_peer.data_ptr() for p in range(world)],
        peer_flag_ptrs=[0 if c == rank else peer_flags[c:].data_ptr() for c in range(world)],
        my_flags_ptr=my_flags.data_ptr(), out_ptr=out.data_ptr(), cta_counter_ptr=counter.data_ptr(),
        rows_per_chunk=rows, rank=rank, epoch=epoch)
    gemm(x, w, out=partial, scatter=scatter)
    torch.cuda.synchronize()
    ops.check_status()
    ref = x.float() @ w.float().t()
    mine = ref[rank * rows:(rank + 1) * rows]
    theirs = ref[other * rows:(other + 1) * rows]
    assert ((peer_mem.float() - theirs).abs().max() / theirs.abs().max()) < 6e-3
    want = partial.float() + from_peer.float()
    assert (out.float() - want).abs().max() <= 0.02 * want.abs().max()
    assert ((partial.float() - mine).abs().max() / mine.abs().max()) < 6e-3
    assert peer_flags[other].item() == epoch


def test_bounded_wait_reports_timeout():
    """A flag that nobody sets: the wait gives up after its budget, records the code and the
    context stays usable."""
    import time

    from halite_b200 import ops

    C = ops.ext()
    flags = _i32(2)
    status = ops.status_word(flags.device)
    t0 = time.time()
    C.wait_flags(flags, 1, status)
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 10.0
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status()
    ops.check_status()                      # cleared
    C.signal_flags([flags.data_ptr(), flags[1:].data_ptr()], 1)
    C.wait_flags(flags, 1, status)
    torch.cuda.synchronize()
    ops.check_status()
    assert (torch.ones(4, device="cuda") * 2).sum().item() == 8
