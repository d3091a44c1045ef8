"""Dense 383M decoder trained with the SOAP optimizer (Adam in Shampoo's eigenbasis) in place of
AdamW; plain data parallelism because the preconditioner needs whole weight matrices. Takes the
place of the reference's configs/lm/scale_383m_shampoo.py, which names an external
distributed-Shampoo package."""

from functools import partial

from halite_b200.conf import call
from halite_b200.optim.soap import SOAP
from halite_b200.parallel.parallelize import parallelize

from ..models.scaling.base import transformer
from .base import max_length, n_vocab, pretrain

lr = 1e-3
conf = call[pretrain](call[transformer](
    vocab_size=n_vocab, dim=1024, n_heads=8, head_dim=128, n_layers=23, intermediate_size=call[int](1024 * 3.5),
    max_position_embeddings=max_length, softcap=0, post_norm=False, attention_processor="torch"),
    lr=lr, optimizer=partial(SOAP, lr=lr, betas=(0.9, 0.95), weight_decay=0.1, precondition_frequency=10,
                             max_precond_dim=8192))
conf.model.wrapper = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32", data_parallel="ddp")
