"""Dense 662M decoder (dim 1024, 23 layers, wide 7168 SwiGLU) on DCLM."""

from halite_b200.conf import call

from ..models.scaling.base import transformer
from .base import max_length, n_vocab, pretrain

conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=1024, n_heads=8, head_dim=128, n_layers=23, intermediate_size=call[int](1024 * 3.5 * 2),
    max_position_embeddings=max_length, softcap=0, post_norm=False, attention_processor="torch"), lr=1e-3)
