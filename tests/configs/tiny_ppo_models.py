"""Tiny stand-in for a model-zoo file with `model`, `model_body`, `model_infer` and `model_conf`
(what the PPO iteration benchmark reads)."""

import os
from functools import partial

from torch import nn

from halite_b200.conf import call, field
from halite_b200.conf.loader import load_module

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_zoo = load_module(os.path.join(_ROOT, "configs/models/transformer.py"))

conf = field()
_t = field(vocab_size=128, dim=64, n_heads=4, head_dim=16, n_layers=2, intermediate_size=176, context_len=128,
           n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True)
conf.model = call[_zoo.transformer](**_t, init=partial(nn.init.normal_, std=0.05))
conf.model_body = call[_zoo.transformer](**_t, use_head=False, init=partial(nn.init.normal_, std=0.05))
conf.model_infer = call[_zoo.transformer_infer](**_t, infer="paged")
conf.model_conf = field(**_t, dtype="float32")
