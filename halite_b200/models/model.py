"""Mixin with `dtype` / `device` of a module's first parameter (reference: transformers/model.py)."""

from __future__ import annotations

import torch


class ModelMixin:
    @property
    def device(self):
        for p in self.parameters():
            return p.device
        for b in self.buffers():
            return b.device
        return torch.device("cpu")

    @property
    def dtype(self):
        for p in self.parameters():
            if p.is_floating_point():
                return p.dtype
        return torch.get_default_dtype()
