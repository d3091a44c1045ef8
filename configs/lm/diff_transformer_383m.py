"""Differential Transformer, 383M (dim 1024, 4 paired heads, 23 layers) on DCLM."""

from halite_b200.conf import call

from ..models.diff_transformer import diff_transformer
from .base import max_length, n_vocab, pretrain

conf = call[pretrain](call[diff_transformer](
    vocab_size=n_vocab, dim=1024, n_heads=4, n_layers=23, intermediate_size=call[int](1024 * 3.5),
    max_position_embeddings=max_length, softcap=0, post_norm=False, attention_processor="torch"), lr=1e-3)
