"""`TransformerDecoder`: embedding -> blocks -> final norm -> head (reference:
transformers/transformer.py:21-418). Module and state-dict names match the reference
(`embedding.embed_input_ids`, `blocks.{i}.self_attention.module.q`, `post_blocks.module`,
`head.linear`), so checkpoints interchange.
"""

from __future__ import annotations


import torch
from torch import nn, utils

from halite_b200.ops import linear as ops_linear
from halite_b200.models.container import ModuleDict
from halite_b200.models.generation import GenerationMixin
from halite_b200.models.model import ModelMixin
from halite_b200.models.types import TransformerDecoderOutput


class TransformerDecoder(nn.Module, ModelMixin, GenerationMixin):
    def __init__(self, embedding, post_embed=None, attention_mask=None, pos_embed=None, blocks=None,
                 post_blocks=None, head=None, tie_embeds=False, use_position_ids=False,
                 attention_processor="native", flex_attention_processor=None, config=None):
        super().__init__()
        self.embedding = embedding
        self.post_embed = post_embed
        self.attention_mask = attention_mask
        self.pos_embed = pos_embed
        self.pos_embed_attention_bias = getattr(pos_embed, "attention_bias", False)
        self.pos_embed_layer_shared = getattr(pos_embed, "layer_shared", True)
        self.blocks = ModuleDict()
        for i, block in enumerate(blocks or []):
            self.blocks[str(i)] = block
        self.post_blocks = post_blocks
        self.head = head
        self.use_position_ids = use_position_ids
        self.attention_processor = attention_processor
        self.flex_attention_processor = flex_attention_processor
        self.tie_embeds = tie_embeds
        if tie_embeds and self.head is not None:
            self.head.tie_weight(self.embedding.embed_weight)
        self.gradient_checkpointing = 0
        self.adapters = None
        self.cache_manager = None
        self.config = config
        self.block_hooks = None   # set by the FSDP layer: (pre_block(i, x) -> x, post_block(i, x, residual) -> (x, residual))

    # ------------------------------------------------------------------ state
    def state_dict(self, *args, **kwargs):
        sd = super().state_dict(*args, **kwargs)
        if self.tie_embeds and self.head is not None:
            prefix = kwargs.get("prefix", args[1] if len(args) > 1 else "")
            sd.pop(prefix + "head." + self.head.tie_weight_key, None)
        return sd

    def load_state_dict(self, state_dict, strict=True, assign=False):
        if self.tie_embeds and self.head is not None:
            state_dict = dict(state_dict)
            state_dict["head." + self.head.tie_weight_key] = state_dict[
                "embedding." + self.embedding.tie_weight_key]
        out = super().load_state_dict(state_dict, strict, assign)
        if self.tie_embeds and self.head is not None and assign:
            self.head.tie_weight(self.embedding.embed_weight)
        return out

    def to_empty(self, *args, **kwargs):
        if getattr(self, "_hb_fsdp", None) is not None:
            return self  # parameters already live in the sharding layer's device buffers
        super().to_empty(*args, **kwargs)
        if self.tie_embeds and self.head is not None:
            self.head.tie_weight(self.embedding.embed_weight)
        return self

    def init_weights(self, device=None):
        def visit(module):
            if hasattr(module, "init_weights") and module is not self:
                module.init_weights()

        for child in self.children():
            child.apply(visit)
        self.init_buffers(device)

    def init_buffers(self, device=None):
        def visit(module):
            if hasattr(module, "init_buffers") and module is not self:
                module.init_buffers(device)

        for child in self.children():
            child.apply(visit)

    def add_adapter(self, name, keys):
        if self.adapters is None:
            self.adapters = {}
        self.adapters[name] = keys

    def gradient_checkpointing_enable(self, n_layer=1, stride=1, ops=False):
        """Activation checkpointing. `n_layer` > 0: blocks are recomputed in groups of `n_layer`
        (1 = every block on its own); with `stride` k only every k-th block is recomputed and the
        others keep their activations (the "selective layer" form). `ops=True` is the selective
        per-op form: inside every block the attention half keeps what it saved and the feed-forward
        half, whose gate / up / activation tensors are most of a block's activation memory, is
        recomputed from its normalised input (reference: transformers/parallelize.py:64-127)."""
        self.gradient_checkpointing = int(n_layer)
        self.checkpoint_stride = max(1, int(stride))
        for block in self.blocks.values():
            block.checkpoint_ff = bool(ops)

    def enable_input_require_grads(self):
        def hook(module, input, output):
            output.requires_grad_(True)

        self._require_grads_hook = self.embedding.get_input_embeddings().register_forward_hook(hook)

    def disable_input_require_grads(self):
        self._require_grads_hook.remove()

    # ------------------------------------------------------------------ forward helpers
    def get_pos_embed(self, pos_embed, attention_mask, query_length, position_ids, device, dtype):
        if self.pos_embed_attention_bias:
            return pos_embed(attention_mask)
        return pos_embed(position_ids, query_length, None, device, dtype)

    def get_attention_mask(self, attention_mask, batch, query_length, key_length, device):
        """[B, K] padding mask (1 = real) -> boolean [B,1,Q,K], True where blocked."""
        extra = None
        if self.attention_mask is not None:
            extra = self.attention_mask(batch, query_length, key_length, device)
        if attention_mask.ndim < 4:
            blocked = ~attention_mask[:, None, None, :].to(torch.bool)
            blocked = blocked.expand(batch, 1, query_length, key_length)
        else:
            blocked = attention_mask
        return blocked if extra is None else blocked | extra

    def _forward_tp(self, tp, input_ids, position_ids, target):
        """Tensor-parallel causal-LM forward: activations between blocks are token shards
        [1, tokens / tp, dim]; the loss is computed vocabulary-parallel."""
        from halite_b200.parallel import tensor_parallel as TP

        B, S = input_ids.shape
        tp.batch_shape = (B, S)
        emb = self.embedding.get_input_embeddings()
        out = TP.vocab_parallel_embedding(input_ids, emb.weight, tp)
        mult = getattr(self.embedding, "multiplier", None)
        if mult is not None:
            out = out * mult
        out = out.unsqueeze(0)
        if self.use_position_ids and position_ids is None:
            position_ids = torch.arange(S, device=out.device).unsqueeze(0)
        pos_emb = None
        if self.pos_embed is not None and not self.pos_embed_attention_bias:
            pos_emb = self.pos_embed(position_ids, S, None, out.device, out.dtype)
        hooks = self.block_hooks
        residual = None
        for key, block in self.blocks.items():
            i = int(key)
            if hooks is not None:
                out = hooks[0](i, out)
            out, residual, _, _ = block(out, residual, None, None, pos_emb=pos_emb, use_cache=False)
            if hooks is not None:
                out, residual = hooks[1](i, out, residual)
        if hooks is not None:
            out = hooks[0](len(self.blocks), out)
        if self.post_blocks is not None:
            out = self.post_blocks(out)
        hidden = TP.gather_rows(out.reshape(-1, out.shape[-1]), tp)          # [B*S, dim]
        if self.head is None:
            return TransformerDecoderOutput(last_hidden_state=hidden.view(B, S, -1))
        weight = self.head.weight
        if target is not None:
            losses = TP.vocab_parallel_cross_entropy(hidden, weight, target.reshape(-1), tp,
                                                     getattr(self.head, "ignore_index", -100))
            loss = losses.mean()
            return TransformerDecoderOutput(loss=loss, loss_dict={"cross entropy": loss.detach()})
        local = ops_linear(hidden, weight)                                   # [B*S, vocab / tp]
        logits = TP.gather_cols(local, tp).view(B, S, -1)
        return TransformerDecoderOutput(logits=logits)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, images=None, cache=None,
                use_cache=False, output_hidden_states=False, bidirection_ids=None,
                document_offsets=None, target=None, unpad_params=None):
        tp = getattr(self, "_hb_tp", None)
        if tp is not None:
            return self._forward_tp(tp, input_ids, position_ids, target)
        emb_in = {}
        if input_ids is not None:
            emb_in["input_ids"] = input_ids
        if images is not None:
            emb_in["images"] = images
        out = self.embedding(**emb_in)
        if self.post_embed is not None:
            out = self.post_embed(out)
        if cache is None:
            cache = [None] * len(self.blocks)
        query_length = out.shape[1]
        past = 0
        if cache and cache[0] is not None:
            past = cache[0].length if hasattr(cache[0], "length") else cache[0][0].shape[1]
        key_length = query_length + past

        if self.use_position_ids and position_ids is None:
            position_ids = torch.arange(past, past + query_length, device=out.device).unsqueeze(0)

        attention_bias = None
        pos_emb = None
        if self.pos_embed is not None and self.pos_embed_layer_shared:
            pe = self.get_pos_embed(self.pos_embed, attention_mask, key_length, position_ids,
                                    out.device, out.dtype)
            if self.pos_embed_attention_bias:
                attention_bias = pe
            else:
                pos_emb = pe

        mask = None
        if attention_mask is not None and unpad_params is None:
            mask = self.get_attention_mask(attention_mask, out.shape[0], query_length, key_length,
                                           out.device)
        if self.flex_attention_processor is not None:
            mask = self.flex_attention_processor(
                batch=out.shape[0], q_len=query_length, kv_len=key_length,
                bidirection_ids=bidirection_ids, position_ids=position_ids,
                document_offsets=document_offsets)

        next_caches, aux_outputs, hidden = [], [], []
        residual = None
        hooks = self.block_hooks
        n_blocks = len(self.blocks)

        if self.gradient_checkpointing > 0 and self.training:
            step = self.gradient_checkpointing
            stride = getattr(self, "checkpoint_stride", 1)
            for start in range(0, n_blocks, step):
                mods = [self.blocks[str(i)] for i in range(start, min(start + step, n_blocks))]

                def run(x, res, mods=mods, start=start):
                    for j, m in enumerate(mods):
                        if hooks is not None:
                            x = hooks[0](start + j, x)
                        x, res, _, _ = m(x, res, mask, attention_bias, pos_emb, None, False, unpad_params)
                        if hooks is not None:
                            x, res = hooks[1](start + j, x, res)
                    return x, res

                if (start // step) % stride == 0:
                    out, residual = utils.checkpoint.checkpoint(run, out, residual, use_reentrant=False)
                else:
                    out, residual = run(out, residual)
        else:
            for key, block in self.blocks.items():
                index = int(key)
                if output_hidden_states:
                    hidden.append(out)
                if hooks is not None:
                    out = hooks[0](index, out)
                out, residual, next_cache, aux = block(
                    out, residual, mask, attention_bias, pos_emb=pos_emb, use_cache=use_cache,
                    cache=cache[index], unpad_params=unpad_params)
                if hooks is not None:
                    out, residual = hooks[1](index, out, residual)
                if use_cache:
                    if hasattr(cache, "update"):      # a cache manager keeps its own per-layer state
                        cache.update(index, next_cache)
                    else:
                        next_caches.append(next_cache)
                aux_outputs.append(aux)
            if use_cache and hasattr(cache, "update"):
                next_caches = cache

        if hooks is not None:
            out = hooks[0](n_blocks, out)      # announces the output side (final norm + head)
        if self.post_blocks is not None:
            out = self.post_blocks(out, residual) if residual is not None else self.post_blocks(out)
        if output_hidden_states:
            hidden.append(out)

        if self.head is None:
            return TransformerDecoderOutput(last_hidden_state=out, hidden_states=hidden,
                                            cache=next_caches, aux_outputs=aux_outputs)
        if target is not None:
            loss, loss_dict = self.head(out, target)
            return TransformerDecoderOutput(loss=loss, loss_dict=loss_dict, hidden_states=hidden,
                                            cache=next_caches, aux_outputs=aux_outputs)
        return TransformerDecoderOutput(logits=self.head(out), hidden_states=hidden, cache=next_caches,
                                        aux_outputs=aux_outputs, last_hidden_state=None)
