"""Tokens/s and model-FLOPs utilisation of a training loop, measured on the device.

A CUDA event is recorded on the compute stream at every log step; the time between two log
steps is read when the later event has completed (the log step already reads the loss, so no
extra synchronisation is added). MFU divides model FLOPs (6 per matmul parameter and token, plus
the attention score / value products) by a peak that defaults to B200's nominal dense bf16 rate
and can be set with `HB_PEAK_TFLOPS` (for example to a measured cuBLAS rate).
"""

from __future__ import annotations

import os
import time

import torch

B200_BF16_DENSE_TFLOPS = 2250.0


def model_flops_per_token(model, seq_len: int, causal: bool = True) -> float:
    """Forward + backward FLOPs per token: 6 x parameters that sit in matmuls (embedding lookups
    excluded, a tied head counted once) + attention (12 x layers x seq x width, halved when causal)."""
    n_matmul = 0
    seen = set()
    embed_ids = set()
    for mod in model.modules():
        if isinstance(mod, torch.nn.Embedding) or type(mod).__name__.endswith("Embedding"):
            for p in mod.parameters(recurse=False):
                embed_ids.add(id(p))
    tied_head = getattr(model, "tie_embeds", False)
    for p in model.parameters():
        if id(p) in seen or p.ndim < 2:
            continue
        seen.add(id(p))
        if id(p) in embed_ids and not tied_head:
            continue
        n_matmul += p.numel()
    blocks = getattr(model, "blocks", None)
    n_layers = len(blocks) if blocks is not None else 0
    width = 0
    conf = getattr(model, "config", None)
    for name in ("dim", "hidden_size"):
        width = width or int(getattr(conf, name, 0) or getattr(model, name, 0) or 0)
    if not width and n_layers:
        for p in model.parameters():
            if p.ndim == 2:
                width = p.shape[1]
                break
    attn = 12.0 * n_layers * seq_len * width * (0.5 if causal else 1.0)
    return 6.0 * n_matmul + attn


class ThroughputMeter:
    def __init__(self, flops_per_token: float | None, world_size: int = 1, device=None):
        self.flops_per_token = flops_per_token
        self.world = world_size
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.peak = float(os.environ.get("HB_PEAK_TFLOPS", B200_BF16_DENSE_TFLOPS)) * 1e12
        self._mark = None
        self._tokens = 0

    def add(self, tokens_this_rank: int):
        self._tokens += int(tokens_this_rank)

    def _now(self):
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def lap(self):
        """Call at a log step (after the loss was read, so the stream is drained up to it).
        Returns {"tokens_per_s": whole job, "tokens_per_s_per_gpu", "mfu"} or {} on the first call."""
        now = self._now()
        out = {}
        if self._mark is not None and self._tokens > 0:
            if self.cuda:
                now.synchronize()
                seconds = self._mark.elapsed_time(now) / 1e3
            else:
                seconds = now - self._mark
            if seconds > 0:
                per_gpu = self._tokens / seconds
                out = {"tokens_per_s": per_gpu * self.world, "tokens_per_s_per_gpu": per_gpu}
                if self.flops_per_token:
                    out["tflops_per_gpu"] = per_gpu * self.flops_per_token / 1e12
                    out["mfu"] = per_gpu * self.flops_per_token / self.peak
        self._mark = now
        self._tokens = 0
        return out
