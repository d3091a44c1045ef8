"""Differential Transformer, large (dim 1536, 8 paired heads, 24 layers, soft-cap 50, post-norm),
30k steps at learning rate 6e-4 on DCLM."""

from halite_b200.conf import call

from ..models.diff_transformer import diff_transformer
from .base import max_length, n_vocab, pretrain

conf = call[pretrain](call[diff_transformer](
    vocab_size=n_vocab, dim=1536, n_heads=8, n_layers=24, intermediate_size=call[int](1536 * 3.5),
    max_position_embeddings=max_length, softcap=50.0, post_norm=True, attention_processor="torch"),
    lr=6e-4, max_iter=30000)
