"""Scaling series, large: dim 1536, 16 heads of 96, 24 layers, soft-cap 50, post-norm; 30k steps
at learning rate 6e-4."""

from halite_b200.conf import call

from ...models.scaling.base import transformer
from ..base import max_length, n_vocab, pretrain

conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=1536, n_heads=16, head_dim=1536 // 16, n_layers=24,
    intermediate_size=call[int](1536 * 3.5), max_position_embeddings=max_length, softcap=50.0, post_norm=True,
    attention_processor="torch"), lr=6e-4, max_iter=30000)
