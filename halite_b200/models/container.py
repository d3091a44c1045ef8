"""Containers (reference: transformers/container.py): a ModuleDict whose repr folds runs of
identical layers, and a MultiModule that fans one input out to several modules."""

from __future__ import annotations

from torch import nn


class ModuleDict(nn.ModuleDict):
    def __repr__(self):
        lines, items = [], list(self._modules.items())
        i = 0
        while i < len(items):
            key, mod = items[i]
            text = repr(mod)
            j = i
            while j + 1 < len(items) and repr(items[j + 1][1]) == text:
                j += 1
            name = f"({key})" if j == i else f"({key}-{items[j][0]}) {j - i + 1} x"
            body = "\n  ".join(text.split("\n"))
            lines.append(f"  {name}: {body}")
            i = j + 1
        return self._get_name() + "(\n" + "\n".join(lines) + "\n)"


class MultiModule(nn.Module):
    def __init__(self, **modules):
        super().__init__()
        self.names = list(modules)
        for k, m in modules.items():
            self.add_module(k, m)

    def forward(self, *args, **kwargs):
        return {k: getattr(self, k)(*args, **kwargs) for k in self.names}
