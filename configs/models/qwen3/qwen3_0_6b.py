"""Qwen3-0.6B (28 layers, dim 1024, 16 query / 8 KV heads of 128, SwiGLU 3072, tied embeddings)."""

from functools import partial

from halite_b200.conf import call, field, function
from halite_b200.data.tokenizers.hf import HFTokenizer
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.nn.normalization import RMSNorm
from halite_b200.parallel.parallelize import parallelize

from ..transformer import transformer, transformer_infer
from .checkpoint import to_halite_postprocess, weight_maps

conf = field()

dim = 1024
n_heads = 16
head_dim = 128
context_len = 40960
use_complex_rope = False
qkv_split = True
rms_eps = 1e-6

transformer_config = field(
    vocab_size=151936, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=28, n_key_value_heads=8,
    intermediate_size=3072, rms_norm_epsilon=rms_eps, context_len=context_len,
    pos_embed=RotaryEmbedding(head_dim, context_len, base=1000000, use_rotate_half=True, pre_init=False),
    pos_embed_apply_fn=partial(apply_rotary_emb, use_complex=use_complex_rope),
    qkv_split=qkv_split, gated_ff_split=qkv_split,
    q_norm=RMSNorm(head_dim, eps=rms_eps), k_norm=RMSNorm(head_dim, eps=rms_eps),
    tie_embeds=True,
)

conf.model = call[transformer](**transformer_config)
conf.model_infer = call[transformer_infer](**transformer_config, infer="paged")
conf.model_conf = field(
    vocab_size=151936, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=28, n_key_value_heads=8,
    intermediate_size=3072, rms_norm_epsilon=rms_eps, context_len=context_len, qkv_split=qkv_split,
    gated_ff_split=qkv_split, tie_embeds=True, use_complex_rope=use_complex_rope, dtype="bfloat16")
conf.parallelize = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32")
conf.tokenizer = HFTokenizer()

_maps = {k: v for k, v in weight_maps.items() if k != "lm_head"}     # tied: no separate head
conf.policy = field(weight_maps=_maps, to_halite_postprocess=function(to_halite_postprocess))
