"""Dense 1.7B decoder (dim 2048, 24 layers) on DCLM."""

from halite_b200.conf import call

from ..models.scaling.base import transformer
from .base import max_length, n_vocab, pretrain

conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=2048, n_heads=16, head_dim=128, n_layers=24, intermediate_size=call[int](2048 * 3.5),
    max_position_embeddings=max_length, softcap=0, post_norm=False, attention_processor="torch"), lr=5e-4)
