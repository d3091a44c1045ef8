"""The allocation-free RMSNorm backward, called through its exported C symbol with ctypes and
compared with the regular extension entry point. Collected last on purpose (file name): it must
pass after every other GPU test has used the device, and alone in a fresh process."""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_DIM = 8192


def _lib():
    from halite_b200.csrc.build import SO_PATH, build

    build()
    lib = ctypes.CDLL(SO_PATH)
    fn = lib.hb_rmsnorm_bwd_fixed_scratch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p]
    return fn


def _inputs(rows, dim, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    h = torch.randn(rows, dim, device="cuda", generator=g).bfloat16()
    dy = torch.randn(rows, dim, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(dim, device="cuda", generator=g)).bfloat16()
    dres = torch.randn(rows, dim, device="cuda", generator=g).bfloat16()
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5)
    return dy, h, w, rstd, dres


def _call(fn, dy, h, w, rstd, dres, dx, dw, w_offset=0.0):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
              dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(),
              h.shape[0], h.shape[1], w_offset, stream)


@pytest.mark.parametrize("rows,dim,with_dres", [(4096, 3072, True), (1000, 8192, False), (7, 64, True)])
def test_matches_regular_entry_point_twice_in_a_row(rows, dim, with_dres):
    import halite_b200.ops as ops

    fn = _lib()
    ext = ops.ext()
    # outputs are the caller's: allocate them before the calls under test
    dx = torch.empty(rows, dim, device="cuda", dtype=torch.bfloat16)
    dw = torch.empty(dim, device="cuda", dtype=torch.float32)
    for seed in (1, 2):          # the second call reuses the scratch the first one dirtied
        dy, h, w, rstd, dres = _inputs(rows, dim, seed)
        dres = dres if with_dres else None
        want_dx, want_dw = ext.rmsnorm_bwd(dy, h, w, rstd, dres, 0.0)
        dx.fill_(float("nan"))
        dw.fill_(float("nan"))
        rc = _call(fn, dy, h, w, rstd, dres, dx, dw)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, want_dx)          # same kernel, same inputs
        torch.testing.assert_close(dw, want_dw, rtol=2e-3, atol=2e-2 * (rows ** 0.5) / 64)
        # and against plain fp32 math
        g = dy.float() * w.float()
        xhat = h.float() * rstd[:, None]
        ref_dw = (dy.float() * xhat).sum(0)
        torch.testing.assert_close(dw, ref_dw, rtol=2e-3, atol=2e-2 * (rows ** 0.5) / 64)
        ref_dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
        if dres is not None:
            ref_dx = ref_dx + dres.float()
        torch.testing.assert_close(dx.float(), ref_dx, rtol=2e-2, atol=2e-2)


def test_zero_rows_clears_dw_and_dims_may_change_between_calls():
    """rows == 0 takes the memset path; then the largest dim followed by the smallest one, so the
    second call runs on a scratch that the first left full of unrelated values."""
    import halite_b200.ops as ops

    fn = _lib()
    ext = ops.ext()
    dw = torch.full((64,), float("nan"), device="cuda")
    empty = torch.empty(0, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(64, device="cuda", dtype=torch.bfloat16)
    rstd = torch.empty(0, device="cuda")
    # zero rows: pointers of empty tensors may be NULL, so hand over valid ones
    buf = torch.empty(8, 64, device="cuda", dtype=torch.bfloat16)
    rc = fn(buf.data_ptr(), buf.data_ptr(), w.data_ptr(), dw.data_ptr(), None, buf.data_ptr(), dw.data_ptr(),
            0, 64, 0.0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert float(dw.abs().sum()) == 0.0
    del empty, rstd
    for rows, dim in ((333, MAX_DIM), (5, 64)):
        dy, h, w, rstd, dres = _inputs(rows, dim, 7)
        want_dx, want_dw = ext.rmsnorm_bwd(dy, h, w, rstd, dres, 0.0)
        dx = torch.empty(rows, dim, device="cuda", dtype=torch.bfloat16)
        dw = torch.full((dim,), float("nan"), device="cuda")
        assert _call(fn, dy, h, w, rstd, dres, dx, dw) == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, want_dx)
        torch.testing.assert_close(dw, want_dw, rtol=2e-3, atol=2e-2 * (rows ** 0.5) / 64)
    # rows beyond 31 bits are refused before anything is launched
    assert fn(buf.data_ptr(), buf.data_ptr(), w.data_ptr(), dw.data_ptr(), None, buf.data_ptr(), dw.data_ptr(),
              2 ** 31, 64, 0.0, None) == -1


def test_rejects_sizes_beyond_the_fixed_scratch():
    fn = _lib()
    dim = MAX_DIM + 8
    dy, h, w, rstd, _ = _inputs(4, dim, 0)
    dx = torch.zeros_like(h)
    dw = torch.zeros(dim, device="cuda")
    assert _call(fn, dy, h, w, rstd, None, dx, dw) == -1
    dy, h, w, rstd, _ = _inputs(4, 64, 0)
    assert fn(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr(),
              4, 60, 0.0, None) == -1            # not a multiple of 8
    assert fn(None, h.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr(),
              4, 64, 0.0, None) == -2
    torch.cuda.synchronize()
    assert float(dx.abs().sum()) == 0.0          # nothing was launched
