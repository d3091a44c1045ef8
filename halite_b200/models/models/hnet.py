"""H-Net: a hierarchical byte-level model that learns where to cut its own chunks
(reference: transformers/models/hnet.py:17-392).

One stage = encoder blocks -> router (cosine dissimilarity of neighbouring tokens gives a boundary
probability) -> `chunk` (keep boundary tokens) -> the next stage on the shorter sequence ->
`dechunk` (exponential moving average that spreads each chunk vector over the positions it
stands for) -> straight-through residual -> decoder blocks. The innermost stage is a plain block
stack. Everything runs on one packed row [1, total, dim] described by `cu_seqlens`.

The reference's dechunk borrows mamba-ssm's fused scan. On a GPU the EMA here is a recurrence
kernel of its own (`ops/scan.py:ema_scan`); on CPU it is the same chunked scan the Mamba-2 mixer
uses (`ssd_scan`), with A = -1, dt = log(1 / (1 - p)), B = p, C = 1 and the input divided by dt,
which reduces to  h_t = (1 - p_t) h_{t-1} + p_t x_t.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...nn.normalization import RMSNorm
from ...ops.scan import ema_scan
from ..feedforward import _project
from ..block import TransformerEncoderBlock
from ..generation import GenerationMixin
from ..model import ModelMixin
from ..types import TransformerDecoderOutput, UnpadParams
from .mamba2 import ssd_scan


@dataclass
class RouterOutput:
    boundary_prob: torch.Tensor     # [total, 2]: (no boundary, boundary)
    boundary_mask: torch.Tensor     # [total] bool
    selected_prob: torch.Tensor     # [total, 1] probability of the decision taken


class Router(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.q_proj = nn.Linear(dim, dim, bias=False)
        self.k_proj = nn.Linear(dim, dim, bias=False)
        self.q_proj.weight._no_reinit = True
        self.k_proj.weight._no_reinit = True

    def init_weights(self):
        with torch.no_grad():
            for lin in (self.q_proj, self.k_proj):
                lin.weight.copy_(torch.eye(lin.weight.shape[0], dtype=lin.weight.dtype))

    def forward(self, input: torch.Tensor, cu_seqlens: torch.Tensor | None = None):
        """input [1, total, dim]. The first token of every sequence is always a boundary."""
        x = input[0]
        q = F.normalize(_project(self.q_proj, x[:-1]).float(), dim=-1)
        k = F.normalize(_project(self.k_proj, x[1:]).float(), dim=-1)
        p = torch.clamp((1 - (q * k).sum(-1)) / 2, 0.0, 1.0)
        p = F.pad(p, (1, 0), value=1.0)
        if cu_seqlens is not None:
            p = p.index_fill(0, cu_seqlens[:-1].long(), 1.0)
        prob = torch.stack((1 - p, p), -1)
        selected = prob.argmax(-1)
        mask = selected == 1
        return RouterOutput(prob, mask, prob.gather(-1, selected[:, None]))


def get_seq_idx(cu_seqlens: torch.Tensor, device=None, total: int | None = None):
    """[1, total] int: which packed sequence each position belongs to."""
    cu = cu_seqlens.to(device) if device is not None else cu_seqlens
    total = int(cu[-1]) if total is None else total
    marks = torch.zeros(total + 1, dtype=torch.int32, device=cu.device)
    marks.index_add_(0, cu[1:-1].long(), torch.ones(cu.numel() - 2, dtype=torch.int32, device=cu.device))
    return marks[:total].cumsum(0, dtype=torch.int32)[None]


def get_pos_idx(cu_seqlens: torch.Tensor, device=None, total: int | None = None):
    """[total] int: position of each token inside its own sequence."""
    cu = (cu_seqlens.to(device) if device is not None else cu_seqlens).long()
    total = int(cu[-1]) if total is None else total
    seq = get_seq_idx(cu, total=total)[0].long()
    return torch.arange(total, device=cu.device) - cu[seq]


def chunk(input: torch.Tensor, boundary_mask: torch.Tensor, cu_seqlens: torch.Tensor):
    """Keep the boundary tokens: ([1, kept, dim], cu_seqlens of the kept tokens, longest sequence)."""
    out = input[:, boundary_mask]
    counts = F.pad(boundary_mask.cumsum(0), (1, 0))
    next_cu = counts[cu_seqlens.long()].to(cu_seqlens.dtype)
    next_max = int((next_cu[1:] - next_cu[:-1]).max())
    return out, next_cu, next_max


def dechunk(input: torch.Tensor, boundary_mask: torch.Tensor, boundary_prob: torch.Tensor,
            cu_seqlens: torch.Tensor, n_heads: int = 1, block_size: int = 64,
            dtype: torch.dtype = torch.float32):
    """Smooth the chunk vectors with an EMA whose rate is each chunk's boundary probability, then
    copy every chunk's value to all positions up to the next boundary. `cu_seqlens` describes the
    chunked row (`input` [1, kept, dim]); the result is [1, total, dim]."""
    p = torch.clamp(boundary_prob[..., -1].float(), 1e-4, 1 - 1e-4)[boundary_mask][None]      # [1, kept]
    kept, dim = input.shape[1], input.shape[2]
    plug_back = boundary_mask.cumsum(0) - 1
    if input.is_cuda and not ops.force_reference():
        # one recurrence kernel per direction instead of the chunked formulation
        out = ema_scan(input[0], p[0], cu_seqlens)[None]
        return out[:, plug_back].to(input.dtype)
    seq_idx = get_seq_idx(cu_seqlens, device=input.device, total=kept)
    dt = torch.log(1 / (1 - p))
    x = (input.float() / dt[..., None]).to(dtype)
    A = -torch.ones(n_heads, device=input.device, dtype=torch.float32)
    out, _ = ssd_scan(x.view(1, kept, n_heads, dim // n_heads), dt[..., None].expand(1, kept, n_heads), A,
                      p.to(dtype).view(1, kept, 1, 1), torch.ones(1, kept, 1, 1, device=input.device, dtype=dtype),
                      chunk_size=block_size, seq_idx=seq_idx)
    out = out.reshape(1, kept, dim)
    return out[:, plug_back].to(input.dtype)


def ratio_loss(target_ratio: float, boundary_mask: torch.Tensor, boundary_prob: torch.Tensor):
    """Pushes the share of boundary tokens towards 1 / target_ratio (1.0 at the optimum)."""
    n = float(target_ratio)
    f = boundary_mask.float().mean()
    g = boundary_prob[..., -1].float().mean()
    return n / (n - 1) * ((n - 1) * f * g + (1 - f) * (1 - g))


class Mamba2Block(nn.Module):
    def __init__(self, block: nn.Module, in_proj_init=None, out_proj_init=None):
        super().__init__()
        self.block = block
        self.in_proj_init = in_proj_init
        self.out_proj_init = out_proj_init

    def init_weights(self):
        if hasattr(self.block, "init_weights"):
            self.block.init_weights()
        if self.in_proj_init is not None:
            self.in_proj_init(self.block.in_proj.weight)
        if self.out_proj_init is not None:
            self.out_proj_init(self.block.out_proj.weight)

    def forward(self, input: torch.Tensor, seq_idx: torch.Tensor | None = None):
        return self.block(input, seq_idx=seq_idx)


def _mixer_of(block):
    inner = block.self_attention if isinstance(block, TransformerEncoderBlock) else block
    return getattr(inner, "module", inner)


class HNetBlock(nn.Module):
    """A stack of mixer (+ feed-forward) blocks followed by RMSNorm; Mamba-2 mixers get the
    sequence index, attention mixers the rotary table and the packed-sequence description."""

    def __init__(self, dim: int, blocks: list[nn.Module]):
        super().__init__()
        self.blocks = nn.ModuleList(blocks)
        self.norm = RMSNorm(dim, eps=1e-5)

    def forward(self, input: torch.Tensor, pos_emb: Any = None, unpad_params: UnpadParams | None = None):
        seq_idx = get_seq_idx(unpad_params.cu_seqlens_q, device=input.device, total=input.shape[1])
        out = input
        for block in self.blocks:
            if isinstance(_mixer_of(block), Mamba2Block):
                if isinstance(block, TransformerEncoderBlock):
                    out = block.ff(block.self_attention(out, seq_idx=seq_idx))
                else:
                    out = block(out, seq_idx=seq_idx)
            elif isinstance(block, TransformerEncoderBlock):
                out = block(out, pos_emb=pos_emb, use_cache=False, unpad_params=unpad_params)
            else:
                out = block(out, None, None, pos_emb, None, False, unpad_params)
            if isinstance(out, tuple):
                out = out[0]
        return self.norm(out)


class StraightThrough(torch.autograd.Function):
    """Forward: ones. Backward: identity. Lets the router's confidence receive gradient without
    scaling the activations."""

    @staticmethod
    def forward(ctx, input):
        return torch.ones_like(input)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output


def straight_through(input: torch.Tensor):
    return StraightThrough.apply(input)


class HNet(nn.Module):
    def __init__(self, dim: int, stage_idx: int, main_network: nn.Module, encoder: nn.Module | None = None,
                 decoder: nn.Module | None = None, pos_embed: nn.Module | None = None,
                 prev_dim: int | None = None, n_heads: int = 1, block_size: int = 64,
                 dtype: torch.dtype = torch.float32):
        super().__init__()
        self.dim = dim
        self.stage_idx = stage_idx
        self.encoder = encoder
        self.main_network = main_network
        self.decoder = decoder
        self.pos_embed = pos_embed
        self.innermost = encoder is None
        self.n_heads, self.block_size, self.dtype = n_heads, block_size, dtype
        if not self.innermost:
            self.router = Router(dim)
            self.residual_proj = nn.Linear(dim, dim, bias=False)
        self.pad_dim = None
        if stage_idx > 0 and prev_dim is not None and dim - prev_dim > 0:
            self.pad_dim = nn.Parameter(torch.zeros(dim - prev_dim))

    def init_weights(self, device=None):
        def init(module):
            if module is not self and hasattr(module, "init_weights") and not isinstance(module, HNet):
                module.init_weights()
        for child in self.children():
            if isinstance(child, HNet):
                child.init_weights(device)
            else:
                child.apply(init)
        if not self.innermost:
            nn.init.zeros_(self.residual_proj.weight)
        if self.pad_dim is not None:
            nn.init.zeros_(self.pad_dim)
        self.init_buffers(device)

    def init_buffers(self, device=None):
        def init(module):
            if hasattr(module, "init_buffers") and not isinstance(module, HNet):
                module.init_buffers(device)
        for child in self.children():
            if isinstance(child, HNet):
                child.init_buffers(device)
            else:
                child.apply(init)

    def get_pos_embed(self, unpad_params: UnpadParams, total: int, device, dtype):
        if self.pos_embed is None:
            return None
        positions = get_pos_idx(unpad_params.cu_seqlens_q, device=device, total=total)[None]
        return self.pos_embed(positions, unpad_params.max_length_q, unpad_params, device, dtype)

    def residual_fn(self, out, residual, selected_prob):
        return out * straight_through(selected_prob).to(out.dtype) + residual

    def _body(self, net, x, pos_emb, unpad_params):
        if isinstance(net, HNet):
            return net(x, unpad_params=unpad_params)
        return net(x, pos_emb=pos_emb, unpad_params=unpad_params), ()

    def forward(self, input: torch.Tensor, unpad_params: UnpadParams):
        input_dim = input.shape[-1]
        if self.pad_dim is not None:
            input = torch.cat((input, self.pad_dim.to(input.dtype).expand(*input.shape[:-1], -1)), -1)
        pos_emb = self.get_pos_embed(unpad_params, input.shape[1], input.device, input.dtype)
        if self.innermost:
            out, _ = self._body(self.main_network, input, pos_emb, unpad_params)
            return out[..., :input_dim], ()
        out = self.encoder(input, pos_emb=pos_emb, unpad_params=unpad_params)
        residual = _project(self.residual_proj, out)
        router_out = self.router(out, cu_seqlens=unpad_params.cu_seqlens_q)
        chunked, next_cu, next_max = chunk(out, router_out.boundary_mask, unpad_params.cu_seqlens_q)
        next_params = UnpadParams(next_cu, next_max)
        inner = self.main_network
        if isinstance(inner, HNet):
            chunked, inner_routes = inner(chunked, unpad_params=next_params)
        else:
            inner_pos = self.get_pos_embed(next_params, chunked.shape[1], chunked.device, chunked.dtype)
            chunked, inner_routes = inner(chunked, pos_emb=inner_pos, unpad_params=next_params), ()
        out = dechunk(chunked, router_out.boundary_mask, router_out.boundary_prob, next_cu, self.n_heads,
                      self.block_size, self.dtype)
        out = self.residual_fn(out, residual, router_out.selected_prob[None])
        out = self.decoder(out, pos_emb=pos_emb, unpad_params=unpad_params)
        return out[..., :input_dim], (router_out, *inner_routes)


class HNetDecoder(nn.Module, ModelMixin, GenerationMixin):
    """Byte embedding -> H-Net -> head. `aux_outputs` is one dict per stage with that stage's
    `ratio_loss` (already weighted), so a training step that adds every aux value ending in
    "loss" picks it up; the raw router outputs are on `router_outputs` of the result."""

    def __init__(self, embedding, hnet: HNet, post_blocks=None, head=None, config=None,
                 target_ratios=None, ratio_loss_weight: float = 0.03):
        super().__init__()
        self.embedding = embedding
        self.hnet = hnet
        self.post_blocks = post_blocks
        self.head = head
        self.config = config
        self.target_ratios = target_ratios
        self.ratio_loss_weight = ratio_loss_weight

    def init_weights(self, device=None):
        for name, child in self.named_children():
            if isinstance(child, HNet):
                child.init_weights(device)
            else:
                child.apply(lambda m: m.init_weights() if hasattr(m, "init_weights") else None)

    def forward(self, input_ids: torch.Tensor, unpad_params: UnpadParams | None = None, target=None, **unused):
        out = self.embedding(input_ids=input_ids)
        batch, length, _ = out.shape
        if unpad_params is None:
            out = out.reshape(1, batch * length, -1)
            cu = torch.arange(batch + 1, device=out.device, dtype=torch.int32) * length
            unpad_params = UnpadParams(cu, length)
        out, router_outs = self.hnet(out, unpad_params=unpad_params)
        out = out.view(batch, length, -1)
        if self.post_blocks is not None:
            out = self.post_blocks(out)
        aux = None
        if self.target_ratios is not None and router_outs:
            aux = [{"ratio_loss": self.ratio_loss_weight * ratio_loss(r, ro.boundary_mask, ro.boundary_prob)}
                   for r, ro in zip(self.target_ratios, router_outs)]
        if self.head is None:
            result = TransformerDecoderOutput(last_hidden_state=out, aux_outputs=aux)
        elif target is not None:
            loss, loss_dict = self.head(out, target)
            result = TransformerDecoderOutput(loss=loss, loss_dict=loss_dict, aux_outputs=aux)
        else:
            result = TransformerDecoderOutput(logits=self.head(out), aux_outputs=aux)
        result.router_outputs = router_outs
        return result
