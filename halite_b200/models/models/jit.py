"""JiT: a plain ViT that denoises pixels directly (x-prediction) with adaLN-Zero conditioning on
time + class, 2-D rotary positions, optional in-context class tokens and a bottleneck patch
embedding (reference: transformers/models/jit.py:11-533; Li & He, "Back to Basics: Let Denoising
Generative Models Denoise"). Module names match the reference so checkpoints interchange.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from halite_b200.models.container import ModuleDict
from halite_b200.models.initialize import init_weights


def modulate(input, shift, scale):
    return input * (1 + scale) + shift


def init_normal(std=0.02):
    return lambda w: nn.init.normal_(w, std=std)


def _apply_init(root):
    for m in root.modules():
        if m is not root and hasattr(m, "init_weights"):
            m.init_weights()
    if hasattr(root, "init_weights") and not isinstance(root, (JiT, EncoderJiT)):
        root.init_weights()


class TimeEmbedding(nn.Module):
    """Scalar time -> sinusoidal ("positional") or random-Fourier features -> 2-layer MLP."""

    def __init__(self, dim, freq_embed_dim=256, embed_type="positional", use_mlp=True, scale=1):
        super().__init__()
        self.dim, self.freq_embed_dim, self.embed_type = dim, freq_embed_dim, embed_type
        self.mlp = nn.Sequential(nn.Linear(freq_embed_dim, dim), nn.SiLU(), nn.Linear(dim, dim)) if use_mlp else None
        if embed_type == "fourier":
            self.register_buffer("freqs", torch.randn(freq_embed_dim // 2) * scale)

    def init_weights(self):
        if self.mlp is not None:
            for i in (0, 2):
                nn.init.normal_(self.mlp[i].weight, std=0.02)
                nn.init.zeros_(self.mlp[i].bias)

    def positional_embed(self, t, max_period=10000):
        half = self.freq_embed_dim // 2
        freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float64, device=t.device) / half)
        args = t[:, None].double() * freqs[None]
        emb = torch.cat((args.cos(), args.sin()), -1)
        if self.freq_embed_dim % 2:
            emb = torch.cat((emb, torch.zeros_like(emb[:, :1])), -1)
        return emb

    def fourier_embed(self, t):
        args = torch.outer(t.double(), 2 * math.pi * self.freqs.double())
        return torch.cat((args.cos(), args.sin()), 1)

    def forward(self, t):
        if self.embed_type == "positional":
            out = self.positional_embed(t, self.dim)
        elif self.embed_type == "fourier":
            out = self.fourier_embed(t)
        else:
            raise ValueError(f"Unknown embed type: {self.embed_type}")
        out = out.to(t.dtype)
        if self.mlp is not None:
            out = self.mlp(out.to(self.mlp[0].weight.dtype))
        return out


class LabelEmbedding(nn.Module):
    """Class embedding with one extra row (index n_labels) for the unconditional class."""

    def __init__(self, n_labels, dim):
        super().__init__()
        self.n_labels = n_labels
        self.embed = nn.Embedding(n_labels + 1, dim)

    def init_weights(self):
        nn.init.normal_(self.embed.weight, std=0.02)

    def forward(self, condition, is_uncond=None):
        if is_uncond is not None:
            condition = torch.where(is_uncond, torch.full_like(condition, self.n_labels), condition)
        return self.embed(condition)


def get_1d_sincos_pos_embed(dim, pos):
    omega = 1.0 / 10000 ** (torch.arange(dim // 2, dtype=torch.float64) / (dim / 2))
    out = torch.outer(pos.reshape(-1).double(), omega)
    return torch.cat((out.sin(), out.cos()), 1)


class SinusoidalEmbedding(nn.Module):
    """Fixed 2-D sin/cos position table added to patch tokens."""

    def __init__(self, dim, grid_size, max_position_embeddings=None):
        super().__init__()
        self.dim, self.grid_size = dim, grid_size
        self.register_buffer("pos_embed", torch.zeros(1, grid_size * grid_size, dim), persistent=False)

    def init_weights(self):
        g = torch.arange(self.grid_size, dtype=torch.float64)
        yy, xx = torch.meshgrid(g, g, indexing="ij")
        emb = torch.cat((get_1d_sincos_pos_embed(self.dim // 2, xx), get_1d_sincos_pos_embed(self.dim // 2, yy)), 1)
        self.pos_embed.copy_(emb.unsqueeze(0))

    def forward(self, input):
        return input + self.pos_embed[:, : input.shape[1]].to(input.dtype)


def rotate_half(x):
    a, b = x.chunk(2, -1)
    return torch.cat((-b, a), -1)


class VisionRoPE(nn.Module):
    """Axial 2-D rotary table over a `max_position_embeddings`^2 grid: half of each head rotates
    with the row index, half with the column; `n_label_tokens` leading tokens are left
    unrotated (cos 1, sin 0)."""

    def __init__(self, dim, max_position_embeddings, n_label_tokens=0, theta=10000):
        super().__init__()
        self.dim, self.theta = dim, theta
        self.max_position_embeddings, self.n_label_tokens = max_position_embeddings, n_label_tokens
        n = max_position_embeddings ** 2 + n_label_tokens
        self.register_buffer("freqs_cos", torch.empty(n, 1, dim * 2))
        self.register_buffer("freqs_sin", torch.empty(n, 1, dim * 2))

    def init_weights(self):
        inv = 1.0 / self.theta ** (torch.arange(0, self.dim, 2)[: self.dim // 2].float() / self.dim)
        ang = torch.outer(torch.arange(self.max_position_embeddings, dtype=torch.float32), inv)
        ang = torch.repeat_interleave(ang, 2, dim=1)                         # [G, dim]
        g = ang.shape[0]
        grid = torch.cat((ang[:, None].expand(-1, g, -1), ang[None].expand(g, -1, -1)), -1).reshape(g * g, -1)
        cos, sin = grid.cos(), grid.sin()
        if self.n_label_tokens:
            cos = torch.cat((torch.ones(self.n_label_tokens, cos.shape[1]), cos), 0)
            sin = torch.cat((torch.zeros(self.n_label_tokens, sin.shape[1]), sin), 0)
        self.freqs_cos.copy_(cos.unsqueeze(1))
        self.freqs_sin.copy_(sin.unsqueeze(1))

    def forward(self):
        return self.freqs_cos, self.freqs_sin


def apply_vision_rope(query, key, pos_embed):
    cos, sin = pos_embed
    cos, sin = cos.to(query.dtype), sin.to(query.dtype)
    return query * cos + rotate_half(query) * sin, key * cos + rotate_half(key) * sin


class InContextEmbedding(nn.Module):
    """Prepends `n_tokens` copies of the class embedding (plus learned offsets) to the sequence."""

    def __init__(self, dim, n_tokens):
        super().__init__()
        self.n_tokens = n_tokens
        self.in_context_embed = nn.Parameter(torch.zeros(1, n_tokens, dim))

    def init_weights(self):
        nn.init.normal_(self.in_context_embed, std=0.02)

    def forward(self, input, labels):
        tokens = labels.unsqueeze(1).expand(-1, self.n_tokens, -1) + self.in_context_embed.to(labels.dtype)
        return torch.cat((tokens.to(input.dtype), input), 1)


class BottleneckEmbedding(nn.Module):
    def __init__(self, dim, out_dim, linear_init=None):
        super().__init__()
        self.linear = nn.Linear(dim, out_dim)
        self.linear_init = linear_init

    def init_weights(self):
        init_weights(self.linear, self.linear_init)

    def forward(self, input):
        return self.linear(input)


class JiTModulator(nn.Module):
    """adaLN: condition -> `n_factors` per-channel vectors (zero-initialised)."""

    def __init__(self, dim, n_factors):
        super().__init__()
        self.n_factors = n_factors
        self.activation = nn.SiLU()
        self.linear = nn.Linear(dim, n_factors * dim)

    def init_weights(self):
        nn.init.zeros_(self.linear.weight)
        nn.init.zeros_(self.linear.bias)

    def forward(self, input):
        return self.linear(self.activation(input)).unsqueeze(1).chunk(self.n_factors, -1)


class JiTHead(nn.Module):
    """Final adaLN + linear to pixels, un-patchified to [B, C, H, W]."""

    def __init__(self, norm, modulator, dim, out_dim, patch_size):
        super().__init__()
        self.out_dim, self.patch_size = out_dim, patch_size
        self.norm, self.modulator = norm, modulator
        self.linear = nn.Linear(dim, patch_size * patch_size * out_dim)

    def init_weights(self):
        nn.init.zeros_(self.linear.weight)
        nn.init.zeros_(self.linear.bias)
        if getattr(self.norm, "weight", None) is not None:
            nn.init.ones_(self.norm.weight)

    def forward(self, input, labels):
        shift, scale = self.modulator(labels)
        out = self.linear(modulate(self.norm(input), shift, scale))
        b, n, _ = input.shape
        side, p = int(math.isqrt(n)), self.patch_size
        out = out.reshape(b, side, side, p, p, self.out_dim).permute(0, 5, 1, 3, 2, 4)
        return out.reshape(b, self.out_dim, side * p, side * p)


class JiTBlock(nn.Module):
    def __init__(self, modulator, norm_attn, self_attention, norm_ff, ff):
        super().__init__()
        self.modulator = modulator
        self.norm_attn, self.self_attention = norm_attn, self_attention
        self.norm_ff, self.ff = norm_ff, ff

    def init_weights(self):
        for n in (self.norm_attn, self.norm_ff):
            if getattr(n, "weight", None) is not None:
                nn.init.ones_(n.weight)

    def forward(self, input, condition, pos_emb=None):
        sh_a, sc_a, g_a, sh_f, sc_f, g_f = self.modulator(condition)
        attn, _ = self.self_attention(modulate(self.norm_attn(input), sh_a, sc_a), pos_emb=pos_emb)
        out = input + g_a * attn
        return out + g_f * self.ff(modulate(self.norm_ff(out), sh_f, sc_f))


class JiT(nn.Module):
    def __init__(self, embedding, time_embedding, label_embedding, post_embed=None, pos_embed=None, pos_rope=None,
                 in_context_embed=None, in_context_rope=None, in_context_start=0, blocks=None, head=None):
        super().__init__()
        self.embedding, self.time_embedding, self.label_embedding = embedding, time_embedding, label_embedding
        self.post_embed, self.pos_embed, self.pos_rope = post_embed, pos_embed, pos_rope
        self.in_context_embed, self.in_context_rope = in_context_embed, in_context_rope
        self.in_context_start = in_context_start
        self.blocks = ModuleDict({str(i): b for i, b in enumerate(blocks or [])})
        self.head = head

    def init_weights(self, device=None):
        for m in self.modules():
            if m is not self and hasattr(m, "init_weights"):
                m.init_weights()

    def forward(self, input, times, labels):
        out = self.embedding(input)
        if self.post_embed is not None:
            out = self.post_embed(out)
        if self.pos_embed is not None:
            out = self.pos_embed(out)
        label_embed = self.label_embedding(labels)
        cond = self.time_embedding(times) + label_embed
        for key, block in self.blocks.items():
            i = int(key)
            if self.in_context_embed is not None and i == self.in_context_start:
                out = self.in_context_embed(out, label_embed)
            pos_emb = None
            if i < self.in_context_start and self.pos_rope is not None:
                pos_emb = self.pos_rope()
            elif i >= self.in_context_start and self.in_context_rope is not None:
                pos_emb = self.in_context_rope()
            out = block(out, cond, pos_emb=pos_emb)
        if self.in_context_embed is not None:
            out = out[:, self.in_context_embed.n_tokens:]
        return self.head(out, cond) if self.head is not None else out


class EncoderJiT(nn.Module):
    """A (pretrained, optionally frozen) encoder's blocks followed by conditional JiT blocks;
    the first `cond_start_id` JiT blocks see a zero condition."""

    def __init__(self, encoder, time_embedding, label_embedding, in_context_embed, in_context_rope, blocks=None,
                 head=None, cond_start_id=0):
        super().__init__()
        self.embedding = encoder.embedding
        self.time_embedding, self.label_embedding = time_embedding, label_embedding
        self.in_context_embed, self.in_context_rope = in_context_embed, in_context_rope
        self.encoder = encoder
        self.blocks = ModuleDict({str(i): b for i, b in enumerate(blocks or [])})
        self.head = head
        self.cond_start_id = cond_start_id

    def init_weights(self, device=None):
        for part in (self.time_embedding, self.label_embedding, self.in_context_embed, self.in_context_rope,
                     self.blocks, self.head):
            if part is None:
                continue
            for m in part.modules():
                if hasattr(m, "init_weights"):
                    m.init_weights()

    def freeze_encoder(self):
        self.encoder.requires_grad_(False)

    def forward(self, input, times, labels):
        out = self.encoder.embedding(input)
        residual = None
        for block in self.encoder.blocks.values():
            out, residual, _, _ = block(out, residual, None, pos_emb=None, use_cache=False)
        cond = self.time_embedding(times) + self.label_embedding(labels)
        out = self.in_context_embed(out, cond)
        pos_emb = self.in_context_rope()
        zero = cond * 0
        for key, block in self.blocks.items():
            out = block(out, zero if int(key) < self.cond_start_id else cond, pos_emb=pos_emb)
        out = out[:, self.in_context_embed.n_tokens:]
        return self.head(out, cond) if self.head is not None else out


def encoder_jit_block_iterator(model):
    for i, block in model.encoder.blocks.items():
        yield i, block, model.encoder.blocks
    for i, block in model.blocks.items():
        yield i, block, model.blocks
