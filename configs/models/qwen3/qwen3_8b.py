"""Qwen3-8B (36 layers, dim 4096, 32 query / 8 KV heads of 128, SwiGLU 12288, untied head)."""

from functools import partial

from halite_b200.conf import call, field, function
from halite_b200.data.tokenizers.hf import HFTokenizer
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.nn.normalization import RMSNorm
from halite_b200.parallel.parallelize import parallelize

from ..transformer import transformer, transformer_infer
from .checkpoint import to_halite_postprocess, weight_maps

conf = field()

dim, n_heads, head_dim, context_len, rms_eps = 4096, 32, 128, 40960, 1e-6
qkv_split = True

transformer_config = field(
    vocab_size=151936, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=36, n_key_value_heads=8,
    intermediate_size=12288, rms_norm_epsilon=rms_eps, context_len=context_len,
    pos_embed=RotaryEmbedding(head_dim, context_len, base=1000000, use_rotate_half=True, pre_init=False),
    pos_embed_apply_fn=partial(apply_rotary_emb, use_complex=False),
    qkv_split=qkv_split, gated_ff_split=qkv_split,
    q_norm=RMSNorm(head_dim, eps=rms_eps), k_norm=RMSNorm(head_dim, eps=rms_eps),
)

conf.model = call[transformer](**transformer_config)
conf.model_infer = call[transformer_infer](**transformer_config, infer="paged")
conf.model_conf = field(
    vocab_size=151936, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=36, n_key_value_heads=8,
    intermediate_size=12288, rms_norm_epsilon=rms_eps, context_len=context_len, qkv_split=qkv_split,
    gated_ff_split=qkv_split, use_complex_rope=False, dtype="bfloat16")
conf.parallelize = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32")
conf.tokenizer = HFTokenizer()
conf.policy = field(weight_maps=weight_maps, to_halite_postprocess=function(to_halite_postprocess))
