"""`Probe`: distribution statistics of every linear layer's input, weight, output and their
gradients for one training step (reference: utils/probe.py:53-256).

The reference watches `aten.mm` through a dispatch mode; here linears run on this package's
own GEMM, so the probe plugs into `halite_b200.ops.linear.linear` instead: while active, each
call records statistics keyed by the parameter's module path (`blocks.3.ff.module.linear_out`)
and attaches gradient hooks; weight gradients are read from the main-grad buffer (or `.grad`)
when the probe exits. Output: one JSON line per step (+ optional raw tensors).

    with Probe(model, "probe/stats.jsonl") as probe:
        probe.metadata = {"it": step}
        loss = model(x).loss; loss.backward()
"""

from __future__ import annotations

import json
import uuid
from pathlib import Path
from typing import Any

import torch

QUANTILES = [1e-7, 1e-6, 1e-5, 1e-4, 1e-3, 1e-2, 0.05, 0.1, 0.3, 0.5, 0.7, 0.9, 0.95, 0.99, 0.999, 0.9999,
             0.99999, 0.999999, 0.9999999]
_MAX_QUANTILE_ELEMS = 2 ** 24       # torch.quantile's input limit

_active: "Probe | None" = None


def active_probe():
    return _active


@torch.no_grad()
def get_stats(t: torch.Tensor, remove_inf=False) -> dict[str, Any]:
    if not t.is_floating_point():
        return {}
    x = t.detach().flatten()
    if remove_inf:
        x = x[x.abs() < float("inf")]
    x = x.double() if x.dtype is torch.double else x.float()
    mean, std = x.mean(), x.std()
    z = (x - mean) / std
    q = torch.tensor(QUANTILES, device=x.device, dtype=x.dtype)
    return {"shape": tuple(t.shape), "mean": mean, "std": std, "skew": z.pow(3).double().mean(),
            "kurtosis": z.pow(4).double().mean(), "abs.mean": x.abs().mean(), "max": x.max(), "min": x.min(),
            "quantiles": torch.quantile(x[:_MAX_QUANTILE_ELEMS], q)}


def _plain(v):
    if isinstance(v, torch.Tensor):
        return v.tolist()
    if isinstance(v, dict):
        return {k: _plain(x) for k, x in v.items()}
    if isinstance(v, tuple):
        return list(v)
    return v


class Probe:
    def __init__(self, model=None, output_file: str | None = None, save_tensors=False, verbose=False):
        self.output_file = Path(output_file) if output_file is not None else None
        self.save_tensors = save_tensors
        self.verbose = verbose
        self.store: dict[str, dict] = {}
        self.metadata: dict[str, Any] = {}
        self.enabled = False
        self._names: dict[int, str] = {}
        self._weights: dict[str, torch.Tensor] = {}
        self._count: dict[str, int] = {}
        self._tensor_dir = None
        if model is not None:
            self.bind(model)

    def bind(self, model):
        for name, p in model.named_parameters():
            if name.endswith(".weight"):
                self._names[id(p)] = name[: -len(".weight")]
        # fused views (q|k|v, up|gate) are separate tensor objects over the same storage
        for mod_name, mod in model.named_modules():
            for key, view in (getattr(mod, "_hb_fused", None) or {}).items():
                self._names[id(view)] = f"{mod_name}.{key}" if mod_name else key
        return self

    def path_of(self, weight):
        name = self._names.get(id(weight))
        if name is None:
            name = f"linear@{tuple(weight.shape)}"
        n = self._count.get(name, 0)
        self._count[name] = n + 1
        return name if n == 0 else f"{name}#{n}"

    # ------------------------------------------------------------------ called from ops.linear
    def on_linear(self, x, weight, out):
        path = self.path_of(weight)
        self.log_tensor(f"{path}::in", x)
        self.log_tensor(f"{path}::weight", weight)
        self.log_tensor(f"{path}::out", out)
        self._weights[path] = weight
        if out.requires_grad:
            out.register_hook(lambda g, p=path: self.log_tensor(f"{p}::out.g", g))
        if x.requires_grad:
            x.register_hook(lambda g, p=path: self.log_tensor(f"{p}::in.g", g))

    def log_tensor(self, name, tensor, **kwargs):
        self.store[name] = get_stats(tensor, **kwargs)
        if self._tensor_dir is not None:
            torch.save(tensor.detach().cpu(), self._tensor_dir / (name.replace("::", "__").replace("/", "") + ".pt"))

    # ------------------------------------------------------------------ context
    def __enter__(self):
        global _active
        if self.enabled:
            raise RuntimeError("entered probe mode twice")
        self.enabled = True
        _active = self
        if self.output_file is not None:
            self.output_file.parent.mkdir(parents=True, exist_ok=True)
            if self.save_tensors:
                self._tensor_dir = self.output_file.parent / f"tensors-{uuid.uuid4().hex[:8]}"
                self._tensor_dir.mkdir(exist_ok=True)
        return self

    def __exit__(self, *exc):
        global _active
        _active = None
        self.enabled = False
        for path, w in self._weights.items():
            g = getattr(w, "_hb_grad", None)
            if g is None:
                g = w.grad
            if g is not None:
                self.log_tensor(f"{path}::w.g", g)
        self.flush_and_clear()

    def flush_and_clear(self):
        if self.output_file is not None:
            with self.output_file.open("a") as f:
                json.dump({"data": _plain(self.store), "meta": self.metadata, "quantiles": QUANTILES}, f)
                f.write("\n")
        if self._tensor_dir is not None:
            final = self._tensor_dir.parent / "tensors"
            final.mkdir(exist_ok=True)
            name = f"it{int(self.metadata['it']):010}" if "it" in self.metadata else ""
            if not name or (final / name).exists():
                name = f"{name}v{len(list(final.glob(name + 'v*')))}"
            self._tensor_dir.rename(final / name)
            self._tensor_dir = None
        self.last = dict(self.store)
        self.store.clear()
        self._weights.clear()
        self._count.clear()
