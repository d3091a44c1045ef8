"""`Record`: the dictionary that flows through data pipelines (reference: data/record.py:4-75).
Keys under `_meta_` carry bookkeeping (dataset name, sample id); tensors move with `.to()`."""

from __future__ import annotations

import torch


class Record(dict):
    META = "_meta_"

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __setattr__(self, key, value):
        self[key] = value

    @property
    def meta(self):
        return self.setdefault(self.META, {})

    def to(self, *args, **kwargs):
        out = Record()
        for k, v in self.items():
            out[k] = v.to(*args, **kwargs) if isinstance(v, torch.Tensor) else v
        return out

    def pin_memory(self):
        out = Record()
        for k, v in self.items():
            out[k] = v.pin_memory() if isinstance(v, torch.Tensor) else v
        return out

    def slice(self, start, end=None):
        """Rows [start, end) of every batched field."""
        sl = slice(start, end)
        out = Record()
        for k, v in self.items():
            if k == self.META:
                out[k] = v
            elif isinstance(v, (torch.Tensor, list, tuple)):
                out[k] = v[sl]
            else:
                out[k] = v
        return out

    def batch_size(self):
        for k, v in self.items():
            if k != self.META and isinstance(v, (torch.Tensor, list, tuple)):
                return len(v)
        return 0

    def unbind(self, keys=None):
        """One Record per row, restricted to `keys` (all batched fields by default)."""
        keys = [k for k in (keys if keys is not None else self.keys()) if k != self.META]
        n = max((len(self[k]) for k in keys if isinstance(self[k], (torch.Tensor, list, tuple))), default=0)
        rows = []
        for i in range(n):
            r = Record()
            for k in keys:
                v = self[k]
                r[k] = v[i] if isinstance(v, (torch.Tensor, list, tuple)) else v
            rows.append(r)
        return rows
