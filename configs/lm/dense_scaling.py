"""Dense 383M decoder of the scaling series with logit soft-capping 50 and post-norm blocks, on
DCLM (dim 1024, 8 heads, 23 layers)."""

from halite_b200.conf import call

from ..models.scaling.base import transformer
from .base import max_length, n_vocab, pretrain

conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=1024, n_heads=8, head_dim=128, n_layers=23, intermediate_size=call[int](1024 * 3.5),
    max_position_embeddings=max_length, softcap=50.0, post_norm=True, attention_processor="torch"), lr=1e-3)
