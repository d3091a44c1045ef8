"""A tiny byte-level model section (model, paged-inference variant, tokenizer, model_conf) for
tests that need a saved model folder."""

import os
from functools import partial

from torch import nn

from halite_b200.conf import call, field
from halite_b200.conf.loader import load_module
from halite_b200.data.tokenizers import ByteTokenizer
from halite_b200.parallel import parallelize

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_zoo = load_module(os.path.join(_ROOT, "configs/models/transformer.py"))

_t = field(vocab_size=260, dim=64, n_heads=4, head_dim=16, n_layers=2, intermediate_size=176, context_len=256,
           n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True)

conf = field(
    model=call[_zoo.transformer](**_t, init=partial(nn.init.normal_, std=0.05)),
    model_infer=call[_zoo.transformer_infer](**_t, infer="paged"),
    model_conf=field(**_t, dtype="float32"),
    tokenizer=ByteTokenizer(),
    parallelize=partial(parallelize, param_dtype="float32", reduce_dtype="float32"),
)
