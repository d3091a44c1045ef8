"""nGPT, 383M: no weight decay, no warm-up, weights re-normalised after every step."""

from functools import partial

from halite_b200.conf import call
from halite_b200.models.optimizer import ngpt_normalize

from ..models.ngpt import ngpt
from .base import max_length, n_vocab, pretrain

conf = call[pretrain](call[ngpt](
    vocab_size=n_vocab, dim=1024, n_heads=8, n_layers=23, intermediate_size=call[int](1024 * 3.5),
    max_position_embeddings=max_length, softcap=0, attention_processor="torch"),
    lr=1e-3, weight_decay=0, warmup=1, postprocess=partial(ngpt_normalize))
