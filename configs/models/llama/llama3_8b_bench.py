"""Benchmark variant of Llama-3-8B: N(0, 0.02) initialisation, the head replaced by the fused linear
+ cross-entropy module (loss computed in the model; vocab-parallel under tensor parallelism), and
blocks that fold every residual add into the following RMSNorm kernel."""

from functools import partial

from halite_b200.conf import call, field
from halite_b200.models.position import Llama3RoPE, apply_rotary_emb
from torch import nn

from ..transformer import transformer, use_fused_linear_cross_entropy, use_fused_residual

conf = field()

dim = 4096
n_heads = 32
head_dim = dim // n_heads

conf.model = use_fused_residual(use_fused_linear_cross_entropy(
    call[transformer](
        vocab_size=128256,
        dim=dim,
        n_heads=n_heads,
        head_dim=head_dim,
        n_layers=32,
        n_key_value_heads=8,
        intermediate_size=14336,
        rms_norm_epsilon=1e-5,
        context_len=8192,
        pos_embed=Llama3RoPE(head_dim, 8192, use_complex=True),
        pos_embed_apply_fn=partial(apply_rotary_emb, use_complex=True),
        qkv_split=True,
        gated_ff_split=True,
        init=partial(nn.init.normal_, std=0.02),
    )
))
