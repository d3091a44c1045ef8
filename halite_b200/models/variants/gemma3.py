"""Gemma-3 specific pieces (reference: transformers/variants/gemma3.py:7-85): an embedding whose
scale is a non-persistent buffer, the `(1 + w)` RMSNorm, and the projector that turns vision
encoder patches into a fixed number of soft tokens per image."""

from __future__ import annotations

import torch
from torch import nn

from halite_b200.models.embedding import TextEmbedding as _TextEmbedding
from halite_b200.nn.normalization import RMSNorm as _RMSNorm


class TextEmbedding(_TextEmbedding):
    def __init__(self, embed_input_ids, dropout=0, embed_init=None, multiplier=None):
        super().__init__(embed_input_ids, dropout, embed_init)
        if hasattr(self, "multiplier"):
            del self.multiplier
        self.register_buffer("multiplier", torch.tensor(float(multiplier)), persistent=False)

    def forward(self, input_ids):
        word = self.embed_input_ids(input_ids)
        # the scale is rounded to the activation dtype first, as the released weights expect
        word = word * self.multiplier.to(word.dtype)
        return self.dropout(word)


class RMSNorm(_RMSNorm):
    """y = x / rms(x) * (1 + w), w initialised at zero; runs on the fused kernel through the
    base class's `weight_offset`."""

    def __init__(self, dim, eps=1e-6):
        super().__init__(dim, eps=eps, weight_offset=1.0)
        with torch.no_grad():
            self.weight.zero_()

    def init_weights(self):
        with torch.no_grad():
            self.weight.zero_()


class MultiModalProjector(nn.Module):
    def __init__(self, encoder, vision_dim, text_dim, norm_eps, image_size, patch_size, tokens_per_image):
        super().__init__()
        self.encoder = encoder
        self.input_proj = nn.Parameter(torch.zeros(vision_dim, text_dim))
        self.soft_embed_norm = RMSNorm(vision_dim, eps=norm_eps)
        self.patches_per_image = int(image_size // patch_size)
        self.token_per_side = int(tokens_per_image ** 0.5)
        self.kernel_size = self.patches_per_image // self.token_per_side
        self.avg_pool = nn.AvgPool2d(self.kernel_size, stride=self.kernel_size)

    def init_weights(self):
        nn.init.normal_(self.input_proj, std=self.input_proj.shape[0] ** -0.5)

    def forward(self, images):
        feats = self.encoder(images=images).last_hidden_state          # [B, patches, vision_dim]
        dtype = feats.dtype
        b, _, d = feats.shape
        grid = feats.transpose(1, 2).reshape(b, d, self.patches_per_image, self.patches_per_image)
        pooled = self.avg_pool(grid.contiguous()).flatten(2).transpose(1, 2)   # [B, tokens, vision_dim]
        return (self.soft_embed_norm(pooled) @ self.input_proj.to(pooled.dtype)).to(dtype)
