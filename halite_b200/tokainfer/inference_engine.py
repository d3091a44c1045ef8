"""`InferenceEngine` of engine B: the same facade as the in-process engine (`initialize`,
`cleanup`, `load_state_dict`, `infer_batch`) over a manager + model worker pair
(reference: tokainfer/inference_engine.py:30-301, entry.py:10-172).

`placement="inline"` keeps the worker in this process; `placement="process"` spawns it (the model
is then built inside the worker from a picklable `build_model` callable) and talks to it through
multiprocessing queues, so scheduling overlaps with device execution.
"""

from __future__ import annotations

import queue
from collections import deque

from halite_b200.infer.types import InferenceRequest, InferenceResult, ModelConfig
from halite_b200.tokainfer.manager import Manager
from halite_b200.tokainfer.types import Command, ServerConfig
from halite_b200.tokainfer.worker import ModelWorker, worker_main


class _InlineChannel:
    def __init__(self, worker):
        self.worker, self.outputs = worker, deque()

    def send(self, inp):
        self.outputs.append(self.worker.run(inp))

    def recv(self, block=True):
        return self.outputs.popleft() if self.outputs else None

    def command(self, cmd):
        self.worker.handle(cmd)

    def sizes(self):
        return self.worker.num_blocks, self.worker.max_seqs

    def close(self):
        pass


class _ProcessChannel:
    def __init__(self, build_model, model_config, server_config, timeout=600.0):
        import torch.multiprocessing as mp

        ctx = mp.get_context("spawn")
        self.in_q, self.out_q = ctx.Queue(), ctx.Queue()
        self.proc = ctx.Process(target=worker_main, args=(build_model, model_config, server_config, self.in_q, self.out_q),
                                daemon=True)
        self.proc.start()
        self.timeout = timeout
        tag, self.num_blocks, self.max_seqs = self.out_q.get(timeout=timeout)
        assert tag == "ready"

    def send(self, inp):
        self.in_q.put(inp)

    def recv(self, block=True):
        try:
            return self.out_q.get(timeout=self.timeout) if block else self.out_q.get_nowait()
        except queue.Empty:
            if block:
                raise TimeoutError("the model worker did not answer") from None
            return None

    def command(self, cmd):
        self.in_q.put(cmd)
        tag, kind = self.out_q.get(timeout=self.timeout)
        assert tag == "done" and kind == cmd.kind
        if cmd.kind == "initialize":
            _, self.num_blocks, self.max_seqs = self.out_q.get(timeout=self.timeout)

    def sizes(self):
        return self.num_blocks, self.max_seqs

    def close(self):
        if self.proc.is_alive():
            self.in_q.put(Command("shutdown"))
            self.proc.join(timeout=30)
            if self.proc.is_alive():
                self.proc.kill()


class InferenceEngine:
    def __init__(self, model, tokenizer, model_config: ModelConfig, server_config: ServerConfig | None = None,
                 build_model=None):
        self.tokenizer = tokenizer
        self.model_config = model_config
        self.server_config = server_config or ServerConfig()
        if self.server_config.placement == "process":
            if build_model is None:
                raise ValueError("placement='process' needs a picklable build_model callable")
            self.channel = _ProcessChannel(build_model, model_config, self.server_config)
        else:
            self.channel = _InlineChannel(ModelWorker(model, model_config, self.server_config))
        self.initialized = True
        self._new_manager()

    def _new_manager(self):
        num_blocks, max_seqs = self.channel.sizes()
        eos = []
        if self.tokenizer is not None:
            if getattr(self.tokenizer, "eos_id", None) is not None:
                eos.append(self.tokenizer.eos_id)
            eos.extend(getattr(self.tokenizer, "additional_stop_token_ids", None) or [])
        self.manager = Manager(self.server_config, self.tokenizer, num_blocks, max_seqs, self.model_config.context_len,
                               self.channel.send, eos)

    # ------------------------------------------------------------------ lifecycle
    def initialize(self):
        if self.initialized:
            return
        self.channel.command(Command("initialize"))
        self._new_manager()
        self.initialized = True

    def cleanup(self):
        if not self.initialized:
            return
        self.channel.command(Command("cleanup"))
        self.initialized = False

    def load_state_dict(self, state_dict, assign=True):
        if isinstance(self.channel, _ProcessChannel):
            state_dict = {k: v.detach() for k, v in sorted(state_dict.items())}
        self.channel.command(Command("load_state_dict", state_dict))

    def update_weights_broadcast(self, src=0, group=None):
        """Take new weights from rank `src` of `group` with one `dist.broadcast` per parameter,
        written in place into the worker's model (reference: tokainfer/utils.py:774-782). Inline
        placement only: the worker's tensors must be reachable from this process."""
        if not isinstance(self.channel, _InlineChannel):
            raise RuntimeError("broadcast weight updates need placement='inline'")
        self.channel.worker.update_weights_broadcast(src, group)

    def cancel(self, request_ids):
        """Cancel requests by id; safe to call from a callback between scheduling rounds (for
        example the `on_step` hook of `infer_batch`)."""
        return self.manager.cancel(request_ids)

    def shutdown(self):
        self.channel.close()

    @property
    def stats(self):
        return self.manager.stats.calc_stats()

    # ------------------------------------------------------------------ inference
    def _normalise(self, i, req):
        if isinstance(req, str):
            return i, self.tokenizer.encode(req), {}
        if isinstance(req, InferenceRequest):
            return req.id, req.input_ids, req.sampling_params
        if isinstance(req, dict):
            return req.get("id", i), req["input_ids"], req.get("sampling_params", {})
        if len(req) == 2:
            ids, sp = req
            return i, ids, sp
        return req

    def infer_batch(self, requests, on_step=None):
        """Run every request to completion; returns one `InferenceResult` per request (with `n`
        samples each), ordered by request id. `on_step(engine)` runs after every batch of results
        and may call `engine.cancel(...)`."""
        mgr = self.manager
        groups = {}
        for i, req in enumerate(requests):
            rid, ids, sp = self._normalise(i, req)
            if isinstance(ids, str):
                ids = self.tokenizer.encode(ids)
            groups[rid] = (list(ids), mgr.add_request(rid, ids, sp or {}))
        while not mgr.idle():
            mgr.schedule_ahead()
            if mgr.inflight_steps:
                out = self.channel.recv(block=True)
                mgr.process_output(out)
                # drain whatever else has already arrived without blocking
                while mgr.inflight_steps:
                    more = self.channel.recv(block=False)
                    if more is None:
                        break
                    mgr.process_output(more)
                if on_step is not None:
                    on_step(self)
            elif mgr.waiting and not mgr.running:
                mgr.schedule_ahead()
                if not mgr.inflight_steps and not mgr.running:
                    break
        mgr.pop_finished()
        results = []
        for rid, (ids, seqs) in sorted(groups.items(), key=lambda kv: str(kv[0])):
            outs = [getattr(s, "prior_output", []) + s.output_ids for s in seqs]
            lps = [getattr(s, "prior_logprobs", []) + s.output_logprobs for s in seqs]
            results.append(InferenceResult(rid, ids, outs, lps, [s.finish_reason for s in seqs],
                                           [s.cached_tokens for s in seqs]))
            mgr.stats.add_finished_req()
        return results
