"""Depth-stacking study, control: the full 28-layer 900M model (dim 1408, 11 heads, soft-cap 50,
post-norm) trained from scratch for 100k steps at learning rate 0.01."""

from functools import partial

from halite_b200.conf import call
from halite_b200.parallel.fsdp import apply_fsdp

from ...models.scaling.base import transformer
from ..base import max_length, n_vocab, pretrain

conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=1408, n_heads=11, head_dim=128, n_layers=28, intermediate_size=call[int](1408 * 3.5),
    max_position_embeddings=max_length, softcap=50.0, post_norm=True, attention_processor="torch"),
    lr=0.01, weight_decay=1e-4 / 0.01, max_iter=100000, activation_checkpointing=False)
conf.model.wrapper = partial(apply_fsdp, param_dtype="bfloat16", reduce_dtype="float32")
conf.training.gradient_checkpointing = True
