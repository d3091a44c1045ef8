"""`InferenceEngine`: the in-process rollout engine (reference: infer/engine/engine.py:13-106).

    engine = InferenceEngine(model_infer, tokenizer, ModelConfig(...), ServerConfig(...))
    engine.load_state_dict(trainer_model.state_dict())   # live weights, no checkpoint round trip
    results = engine.infer_batch(requests)
    engine.cleanup()        # hand the GPU back to training
    engine.initialize()     # ... and take it again
"""

from __future__ import annotations

import copy
from typing import Any

from torch import nn

from halite_b200.infer.model_runner import ModelRunner
from halite_b200.infer.scheduler import Scheduler
from halite_b200.infer.types import InferenceResult, ModelConfig, ServerConfig


class InferenceEngine:
    def __init__(self, model: nn.Module, tokenizer: Any, model_config: ModelConfig,
                 server_config: ServerConfig | None = None, tp_group=None):
        """`model_config.tp_size` > 1 runs the engine tensor-parallel over `tp_group`: every rank of
        the group constructs the engine, loads the same state dict and calls `infer_batch` with the
        same requests; each keeps its slice of the weights and its KV heads."""
        server_config = server_config or ServerConfig()
        self._ids = 0
        if model_config.tp_size > 1 and getattr(model, "_infer_tp", None) is None:
            import torch.distributed as dist

            from halite_b200.infer.tensor_parallel import apply_infer_tp

            apply_infer_tp(model, dist.get_rank(tp_group), model_config.tp_size, tp_group)
        self.model_runner = ModelRunner(model, model_config, server_config)
        self.scheduler = Scheduler(self.model_runner, tokenizer, server_config)
        self.model_config = model_config
        self.server_config = server_config
        self.tokenizer = tokenizer
        self.initialized = True

    def initialize(self):
        if self.initialized:
            return
        if self.model_runner.kv_pool is None:
            self.model_runner.initialize()
        else:                              # kept resident: every page and request slot is free again
            self.model_runner.reset_pools()
        self.scheduler.initialize()
        self.initialized = True

    def cleanup(self):
        if not self.initialized:
            return
        self.scheduler.cleanup()
        if not self.server_config.keep_resident:
            self.model_runner.cleanup()
        self.initialized = False

    def load_state_dict(self, state_dict, assign=True):
        self.model_runner.load_state_dict(state_dict, assign=assign)

    def load_from_model(self, train_model):
        """Weights straight from a sharded training model (one reshard kernel launch)."""
        self.model_runner.load_from_model(train_model)

    def _new_id(self):
        # a counter, not a random id: tensor-parallel ranks must name (and order) requests alike
        self._ids += 1
        return f"_hb-internal-{self._ids:09d}"

    @property
    def stats(self):
        return self.scheduler.stats

    def infer_batch(self, requests):
        requests = self.scheduler.build_batch_request(requests)
        if not requests:
            return []
        n = requests[0].sampling_params.n
        if any(r.sampling_params.n != n for r in requests):
            raise ValueError("all requests of one infer_batch call must ask for the same number of samples")
        if n == 1:
            done = sorted(self.scheduler.infer_batch(requests), key=lambda x: str(x[0]))
            return [InferenceResult(i, inp, [out], [lp], [why], [cached])
                    for i, inp, out, lp, why, cached in done]
        # n > 1: one zero-token request per prompt seeds the prefix cache, then n copies each
        seeds = []
        for r in requests:
            s = copy.copy(r)
            s.id = self._new_id()
            s.sampling_params = copy.copy(r.sampling_params)
            s.sampling_params.max_new_tokens = 0
            s.output_ids, s.output_logprobs = [], []
            seeds.append(s)
        self.scheduler.infer_batch(seeds)
        owner, copies = {}, []
        for r in requests:
            for _ in range(n):
                c = copy.copy(r)
                c.id = self._new_id()
                c.output_ids, c.output_logprobs = [], []
                owner[c.id] = r.id
                copies.append(c)
        grouped = {}
        for i, inp, out, lp, why, cached in self.scheduler.infer_batch(copies):
            g = grouped.setdefault(owner[i], (inp, [], [], [], []))
            g[1].append(out)
            g[2].append(lp)
            g[3].append(why)
            g[4].append(cached)
        return [InferenceResult(i, *g) for i, g in sorted(grouped.items(), key=lambda x: str(x[0]))]
