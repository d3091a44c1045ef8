"""Input embeddings (reference: transformers/embedding.py:7-139)."""

from __future__ import annotations

from torch import nn


class TextEmbedding(nn.Module):
    def __init__(self, embed_input_ids, dropout=0, embed_init=None, multiplier=None):
        super().__init__()
        self.embed_input_ids = embed_input_ids
        self.dropout = nn.Dropout(dropout)
        self.embed_init = embed_init
        self.multiplier = multiplier
        self.tie_weight_key = "embed_input_ids.weight"

    def init_weights(self):
        if self.embed_init is not None:
            self.embed_init(self.embed_input_ids.weight)

    def get_input_embeddings(self):
        return self.embed_input_ids

    @property
    def embed_weight(self):
        return self.embed_input_ids.weight

    def forward(self, input_ids):
        word = self.embed_input_ids(input_ids)
        if self.multiplier is not None:
            word = word * self.multiplier
        return self.dropout(word)

    def tp_plan(self):
        return {"embed_input_ids": "vocab"}


class MultiModalEmbedding(nn.Module):
    """Text embedding whose rows at `image_mask_token_id` are replaced by image embeddings."""

    def __init__(self, text_embedding, image_embedding, image_mask_token_id):
        super().__init__()
        self.text_embedding = text_embedding
        self.image_embedding = image_embedding
        self.image_mask_token_id = image_mask_token_id

    @property
    def tie_weight_key(self):
        return "text_embedding." + self.text_embedding.tie_weight_key

    @property
    def embed_weight(self):
        return self.text_embedding.embed_weight

    def get_input_embeddings(self):
        return self.text_embedding.get_input_embeddings()

    def init_weights(self):
        pass  # children are visited by the model-level walk

    def forward(self, input_ids, images=None):
        out = self.text_embedding(input_ids)
        if images is None:
            return out
        img = self.image_embedding(images).to(out.dtype)
        mask = (input_ids == self.image_mask_token_id).unsqueeze(-1).expand_as(out)
        return out.masked_scatter(mask, img.reshape(-1, out.shape[-1]))


class PatchEmbedding(nn.Module):
    """Image -> patch tokens, by strided convolution or reshape + linear, then an optional
    position embedding (state-dict names `patch_embedding`, `position_embedding`)."""

    def __init__(self, in_dim, out_dim, patch_size, position_embedding=None, use_conv=False, use_bias=False,
                 patch_embedding_init=None):
        super().__init__()
        self.patch_size = patch_size
        self.use_conv = use_conv
        self.patch_embedding_init = patch_embedding_init
        if use_conv:
            self.patch_embedding = nn.Conv2d(in_dim, out_dim, patch_size, patch_size, bias=use_bias)
        else:
            self.patch_embedding = nn.Linear(in_dim * patch_size * patch_size, out_dim, bias=use_bias)
        self.position_embedding = position_embedding

    def init_weights(self):
        w = self.patch_embedding.weight
        if self.patch_embedding_init is not None:
            self.patch_embedding_init(w)
        else:
            nn.init.xavier_uniform_(w.view(w.shape[0], -1))
        if self.patch_embedding.bias is not None:
            nn.init.zeros_(self.patch_embedding.bias)

    def forward(self, images):
        if self.use_conv:
            out = self.patch_embedding(images).flatten(2).transpose(1, 2)
        else:
            p = self.patch_size
            B, C, H, W = images.shape
            x = images.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
            out = self.patch_embedding(x.reshape(B, (H // p) * (W // p), C * p * p))
        if self.position_embedding is not None:
            out = self.position_embedding(out)
        return out
