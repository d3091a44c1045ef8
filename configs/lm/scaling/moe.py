"""Scaling series, mixture of experts: dim 1024, 24 layers, 64 experts of width 896 with top-8
routing, router z-loss 1e-3 and load-balance loss 1e-2, on the 200B-token Nemotron-CC sample
(reference: configs/lm/scaling/moe.py:12)."""

from halite_b200.conf import call

from ...data.nemotron_cc_200b import conf as data_conf
from ...models.moe_transformer import moe_transformer
from ..base import max_length, n_vocab, pretrain

conf = call[pretrain](call[moe_transformer](
    vocab_size=n_vocab, dim=1024, n_heads=8, n_layers=24, n_experts=64, expert_top_k=8, z_loss=1e-3,
    load_balance_loss=1e-2, intermediate_size=call[int](256 * 3.5), max_position_embeddings=max_length, softcap=0,
    post_norm=False, attention_processor="torch"), lr=1e-3)
conf.data.train = data_conf
conf.data.eval = data_conf
