"""Dense 383M decoder trained with Shampoo (Adam-grafted, inverse square roots of the Kronecker
factors) in place of AdamW; plain data parallelism because the preconditioner needs whole weight
matrices. Same hyperparameters as the reference's configs/lm/scale_383m_shampoo.py:75-90, with the
in-tree optimizer instead of the external distributed-Shampoo package."""

from functools import partial

from halite_b200.conf import call
from halite_b200.optim.shampoo import AdamGraftingConfig, Shampoo
from halite_b200.parallel.parallelize import parallelize

from ..models.scaling.base import transformer
from .base import max_length, n_vocab, pretrain

lr = 1e-3
conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=1024, n_heads=8, head_dim=128, n_layers=23, intermediate_size=call[int](1024 * 3.5),
    max_position_embeddings=max_length, softcap=0, post_norm=False, attention_processor="torch"),
    lr=lr, optimizer=partial(Shampoo, lr=lr, betas=(0.9, 0.95), epsilon=1e-12, max_preconditioner_dim=8192,
                             precondition_frequency=10, use_decoupled_weight_decay=True, inv_root_override=2,
                             grafting_config=AdamGraftingConfig(beta2=0.95, epsilon=1e-08)))
conf.model.wrapper = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32", data_parallel="ddp")
