"""Llama-3-8B (32 layers, dim 4096, 32 query / 8 KV heads, SwiGLU 14336, vocab 128256)."""

from functools import partial

from halite_b200.conf import call, field, function
from halite_b200.data.tokenizers.llama3 import Llama3Tokenizer
from halite_b200.models.position import Llama3RoPE, apply_rotary_emb
from halite_b200.parallel.parallelize import parallelize

from ..transformer import transformer, transformer_infer
from .checkpoint import to_halite_postprocess, weight_maps

conf = field()

dim = 4096
n_heads = 32
head_dim = dim // n_heads
context_len = 8192
use_complex_rope = True
qkv_split = True

transformer_config = field(
    vocab_size=128256,
    dim=dim,
    n_heads=n_heads,
    head_dim=head_dim,
    n_layers=32,
    n_key_value_heads=8,
    intermediate_size=14336,
    rms_norm_epsilon=1e-5,
    context_len=context_len,
    pos_embed=Llama3RoPE(head_dim, context_len, use_scaled_rope=False, use_complex=use_complex_rope),
    pos_embed_apply_fn=partial(apply_rotary_emb, use_complex=use_complex_rope),
    qkv_split=qkv_split,
    gated_ff_split=qkv_split,
)

conf.model = call[transformer](**transformer_config)
conf.model_infer = call[transformer_infer](**transformer_config, infer="paged")
conf.model_conf = field(
    vocab_size=128256, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=32, n_key_value_heads=8,
    intermediate_size=14336, context_len=context_len, rms_norm_epsilon=1e-5,
    use_complex_rope=use_complex_rope, qkv_split=qkv_split, dtype="bfloat16")
conf.parallelize = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32")
conf.tokenizer = Llama3Tokenizer()
conf.policy = field(weight_maps=weight_maps, to_halite_postprocess=function(to_halite_postprocess))
