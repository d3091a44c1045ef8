"""`init_weights(module, init_fn)`: apply a weight initialiser to a linear-like module and
zero its bias (reference: transformers/initialize.py)."""

from __future__ import annotations

from torch import nn


def init_weights(module, init_fn):
    if module is None:
        return
    if isinstance(module, nn.Sequential) and len(module) > 0:
        module = module[0]
    if init_fn is not None and getattr(module, "weight", None) is not None:
        init_fn(module.weight)
    if getattr(module, "bias", None) is not None:
        nn.init.constant_(module.bias, 0)
