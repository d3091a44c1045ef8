"""Inference decoder over flat token batches (reference: infer/transformer.py:8-114). Module
names equal the training decoder's, so a training state dict loads unchanged."""

from __future__ import annotations

from torch import nn

from halite_b200.infer.postprocessor import LogitsProcessor
from halite_b200.models.container import ModuleDict
from halite_b200.models.model import ModelMixin


class InferTransformerDecoder(nn.Module, ModelMixin):
    def __init__(self, embedding, pos_embed=None, blocks=None, post_blocks=None, head=None,
                 tie_embeds=False, use_position_ids=True, attention_processor="paged", post_embed=None,
                 config=None):
        super().__init__()
        self.embedding = embedding
        self.post_embed = post_embed
        self.pos_embed = pos_embed
        self.blocks = ModuleDict()
        for i, b in enumerate(blocks or []):
            self.blocks[str(i)] = b
        self.post_blocks = post_blocks
        self.head = head
        self.tie_embeds = tie_embeds
        if tie_embeds and head is not None:
            self.head.tie_weight(self.embedding.embed_weight)
        self.use_position_ids = use_position_ids
        self.logits_processor = LogitsProcessor()
        self.config = config

    def state_dict(self, *args, **kwargs):
        sd = super().state_dict(*args, **kwargs)
        if self.tie_embeds and self.head is not None:
            sd.pop("head." + self.head.tie_weight_key, None)
        return sd

    def load_state_dict(self, state_dict, strict=True, assign=False):
        if self.tie_embeds and self.head is not None:
            state_dict = dict(state_dict)
            state_dict["head." + self.head.tie_weight_key] = state_dict[
                "embedding." + self.embedding.tie_weight_key]
        out = super().load_state_dict(state_dict, strict, assign)
        if self.tie_embeds and self.head is not None:
            self.head.tie_weight(self.embedding.embed_weight)
        self.pack_weights()
        return out

    def pack_weights(self):
        for m in self.modules():
            if m is not self and hasattr(m, "pack_weights"):
                m.pack_weights()

    def init_weights(self, device=None):
        def visit(m):
            if hasattr(m, "init_weights") and m is not self:
                m.init_weights()

        for child in self.children():
            child.apply(visit)
        self.init_buffers(device)
        self.pack_weights()

    def init_buffers(self, device=None):
        def visit(m):
            if hasattr(m, "init_buffers") and m is not self:
                m.init_buffers(device)

        for child in self.children():
            child.apply(visit)

    def set_kv_pool(self, kv_pool):
        from halite_b200.infer.attention import PagedAttention

        for m in self.modules():
            if isinstance(m, PagedAttention):
                m.kv_pool = kv_pool

    def hidden_states(self, forward_batch):
        out = self.embedding(forward_batch.input_ids)
        if self.post_embed is not None:
            out = self.post_embed(out)
        pos_emb = None
        if self.pos_embed is not None:
            pos_emb = self.pos_embed(forward_batch.positions, forward_batch.max_seq_len, None,
                                     out.device, out.dtype)
        from halite_b200.nn.normalization import RMSNorm

        fused = isinstance(self.post_blocks, RMSNorm) and self.post_blocks.weight is not None and \
            all(getattr(b, "fuses_residual", lambda: False)() for b in self.blocks.values())
        if fused:
            residual = None
            for block in self.blocks.values():
                out, residual = block.forward_fused(out, residual, forward_batch, pos_emb)
            return self.post_blocks(out, residual)[0] if residual is not None else self.post_blocks(out)
        for block in self.blocks.values():
            out = block(out, forward_batch, pos_emb)
        if self.post_blocks is not None:
            out = self.post_blocks(out)
        return out

    def forward(self, forward_batch):
        """Returns fp32 logits of each request's last token: [batch, vocab]."""
        out = self.hidden_states(forward_batch)
        if self.head is None:
            if forward_batch.mode.is_decode():
                return out
            return out.index_select(0, forward_batch.sample_indices)
        return self.logits_processor(out, self.head.weight, forward_batch)
