"""Mamba-2 (state-space duality) mixer in plain PyTorch, with a chunked scan
(the reference takes `Mamba2` and `mamba_chunk_scan_combined` from the mamba-ssm package:
configs/models/hnet.py:89-95, transformers/models/hnet.py:104-121).

Recurrence per head: h_t = exp(A dt_t) h_{t-1} + dt_t B_t x_t^T,  y_t = C_t h_t + D x_t.
`ssd_scan` evaluates it chunk by chunk: inside a chunk the output is a masked, decay-weighted
(C B^T) X product (batched matrix products); between chunks a small state is carried, on a GPU by
one recurrence kernel over the chunk axis (`ops/scan.py:linear_scan_autograd`), on CPU by a loop.
Sequences packed into one row are kept apart by `seq_idx` (no decay path across a sequence boundary).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...ops.scan import linear_scan_autograd
from ..feedforward import _project


def _scan_kernel_for(x):
    """Whether the chunk-to-chunk state passing runs on the recurrence kernel (CUDA tensors)."""
    return x.is_cuda and not ops.force_reference()


def _segsum(x):
    """x [..., T] -> [..., T, T] with out[i, j] = sum_{j < k <= i} x[k] (-inf above the diagonal)."""
    T = x.shape[-1]
    cs = x.cumsum(-1)
    out = cs[..., :, None] - cs[..., None, :]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device))
    return out.masked_fill(~mask, float("-inf"))


def ssd_scan(x, dt, A, B, C, chunk_size=64, seq_idx=None, initial_state=None):
    """x [b, L, H, P], dt [b, L, H] (already positive), A [H] (negative), B, C [b, L, G, N] with
    H % G == 0, seq_idx [b, L] int or None. Returns y [b, L, H, P] (without the D skip term)."""
    b, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    pad = (-L) % chunk_size
    if pad:
        x, dt = F.pad(x, (0, 0, 0, 0, 0, pad)), F.pad(dt, (0, 0, 0, pad))
        B, C = F.pad(B, (0, 0, 0, 0, 0, pad)), F.pad(C, (0, 0, 0, 0, 0, pad))
        if seq_idx is not None:
            seq_idx = F.pad(seq_idx, (0, pad), value=-1)
    Lp = L + pad
    nc = Lp // chunk_size
    f32 = torch.float32
    rep = H // G
    xs = (x.to(f32) * dt.to(f32)[..., None]).view(b, nc, chunk_size, H, P)
    a = (dt.to(f32) * A.to(f32)).view(b, nc, chunk_size, H).permute(0, 3, 1, 2)          # [b,H,nc,Q]
    Bc = B.to(f32).repeat_interleave(rep, 2).view(b, nc, chunk_size, H, N)
    Cc = C.to(f32).repeat_interleave(rep, 2).view(b, nc, chunk_size, H, N)
    a_cum = a.cumsum(-1)
    # ---- inside each chunk
    Lmat = torch.exp(_segsum(a))                                                            # [b,H,nc,Q,Q]
    if seq_idx is not None:
        s = seq_idx.view(b, nc, chunk_size)
        same = (s[:, :, :, None] == s[:, :, None, :])[:, None]                              # [b,1,nc,Q,Q]
        Lmat = Lmat * same
    y_diag = torch.einsum("bclhn,bcshn,bhcls,bcshp->bclhp", Cc, Bc, Lmat, xs)
    # ---- state at the end of each chunk, ignoring earlier chunks
    decay_to_end = torch.exp(a_cum[..., -1:] - a_cum)                                       # [b,H,nc,Q]
    if seq_idx is not None:
        last = s[:, :, -1:]
        decay_to_end = decay_to_end * (s == last)[:, None].to(f32)
    states = torch.einsum("bcshn,bhcs,bcshp->bchpn", Bc, decay_to_end, xs)
    # ---- carry states across chunks: carried[c + 1] = carried[c] * keep[c] + states[c]
    chunk_decay = torch.exp(a_cum[..., -1])                                                 # [b,H,nc]
    keep = chunk_decay
    if seq_idx is not None:
        # the carried state survives a chunk only if the chunk ends in the sequence it began in
        # and began in the sequence the previous chunk ended in
        cont = s[:, :, 0] == s[:, :, -1]                                                    # [b,nc]
        cont = cont & torch.cat((torch.ones_like(cont[:, :1]), s[:, 1:, 0] == s[:, :-1, -1]), 1)
        keep = keep * cont.to(f32)[:, None]
    if initial_state is None and _scan_kernel_for(x):
        # one recurrence kernel over the chunk axis: a row per (batch, head, chunk), P*N channels
        rows = states.permute(0, 2, 1, 3, 4).reshape(b * H * nc, P * N)
        cu = torch.arange(0, b * H * nc + 1, nc, device=x.device, dtype=torch.int32)
        after = linear_scan_autograd(rows, keep.reshape(-1), torch.ones(b * H * nc, device=x.device), cu)
        after = after.view(b, H, nc, P, N)
        prev = F.pad(after[:, :, :-1], (0, 0, 0, 0, 1, 0)).permute(0, 2, 1, 3, 4)           # state entering chunk c
        final_state = after[:, :, -1]
    else:
        if initial_state is None:
            initial_state = states.new_zeros(b, H, P, N)
        carried = [initial_state]
        for c in range(nc):
            carried.append(carried[-1] * keep[:, :, c, None, None] + states[:, c])
        prev = torch.stack(carried[:-1], 1)                                                 # state entering chunk c
        final_state = carried[-1]
    decay_from_start = torch.exp(a_cum)                                                     # [b,H,nc,Q]
    if seq_idx is not None:
        first_prev = torch.cat((s[:, :1, :1], s[:, :-1, -1:]), 1)                           # seq of the carried state
        decay_from_start = decay_from_start * (s == first_prev)[:, None].to(f32)
    y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", Cc, prev, decay_from_start)
    y = (y_diag + y_off).reshape(b, Lp, H, P)[:, :L]
    return y.to(x.dtype), final_state


class GatedRMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x, gate):
        x = x.float() * F.silu(gate.float())
        return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float())


class Mamba2(nn.Module):
    def __init__(self, d_model, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=64,
                 dt_min=1e-3, dt_max=0.1, A_init_range=(1, 16), bias=False, conv_bias=True, **unused):
        super().__init__()
        self.d_model, self.d_state, self.d_conv, self.headdim = d_model, d_state, d_conv, headdim
        self.d_inner = expand * d_model
        self.ngroups, self.chunk_size = ngroups, chunk_size
        self.nheads = self.d_inner // headdim
        self.dt_min, self.dt_max, self.A_init_range = dt_min, dt_max, A_init_range
        d_in_proj = 2 * self.d_inner + 2 * ngroups * d_state + self.nheads
        self.in_proj = nn.Linear(d_model, d_in_proj, bias=bias)
        conv_dim = self.d_inner + 2 * ngroups * d_state
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, d_conv, groups=conv_dim, padding=d_conv - 1, bias=conv_bias)
        self.dt_bias = nn.Parameter(torch.zeros(self.nheads))
        self.A_log = nn.Parameter(torch.zeros(self.nheads))
        self.D = nn.Parameter(torch.ones(self.nheads))
        self.norm = GatedRMSNorm(self.d_inner)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=bias)

    def init_weights(self):
        with torch.no_grad():
            dt = torch.exp(torch.rand(self.nheads) * (math.log(self.dt_max) - math.log(self.dt_min))
                           + math.log(self.dt_min)).clamp(min=1e-4)
            self.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))            # inverse softplus
            self.A_log.copy_(torch.log(torch.empty(self.nheads).uniform_(*self.A_init_range)))
            self.D.fill_(1.0)
            self.norm.weight.fill_(1.0)
            nn.init.kaiming_uniform_(self.conv1d.weight, a=math.sqrt(5))
            if self.conv1d.bias is not None:
                nn.init.zeros_(self.conv1d.bias)

    def forward(self, u, seq_idx=None):
        """u [b, L, d_model]; seq_idx [b, L] marks packed sequences."""
        b, L, _ = u.shape
        zxbcdt = _project(self.in_proj, u)
        z, xBC, dt = torch.split(zxbcdt, [self.d_inner, self.d_inner + 2 * self.ngroups * self.d_state, self.nheads], -1)
        xBC_t = xBC.transpose(1, 2)
        if seq_idx is not None:
            # causal depthwise conv that does not look across sequence boundaries
            taps = []
            for k in range(self.d_conv):
                shifted = F.pad(xBC_t, (k, 0))[..., :L]
                if k:
                    ok = F.pad(seq_idx, (k, 0), value=-1)[..., :L] == seq_idx
                    shifted = shifted * ok[:, None]
                taps.append(shifted * self.conv1d.weight[:, 0, self.d_conv - 1 - k][None, :, None])
            conv = sum(taps)
            if self.conv1d.bias is not None:
                conv = conv + self.conv1d.bias[None, :, None]
        else:
            conv = self.conv1d(xBC_t)[..., :L]
        xBC = F.silu(conv).transpose(1, 2)
        x, B, C = torch.split(xBC, [self.d_inner, self.ngroups * self.d_state, self.ngroups * self.d_state], -1)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -torch.exp(self.A_log.float())
        xh = x.view(b, L, self.nheads, self.headdim)
        y, _ = ssd_scan(xh, dt, A, B.view(b, L, self.ngroups, self.d_state), C.view(b, L, self.ngroups, self.d_state),
                        self.chunk_size, seq_idx)
        y = y.float() + xh.float() * self.D.float()[None, None, :, None]
        y = self.norm(y.reshape(b, L, self.d_inner), z)
        return _project(self.out_proj, y.to(u.dtype))
