"""Model worker of engine B (reference: tokainfer/basic_worker.py:36-259, utils.py ModelRunner):
executes `ModelInput`s — mixed prefill chunks and decode tokens in one flat forward — on the
paged kernels and returns the sampled tokens. It owns the KV pages and the page table; the
manager only ever names page ids and table rows. Decode entries whose token the manager has not
seen yet (scheduling ahead) take their input from the worker's device-side last-token buffer, so
no host round trip sits between consecutive decode steps.
"""

from __future__ import annotations

import torch

from halite_b200.infer.batch import BatchSamplingParams, ForwardBatch, ForwardMode
from halite_b200.infer.model_runner import ModelRunner
from halite_b200.infer.types import ServerConfig as RunnerConfig
from halite_b200.tokainfer.types import Command, ModelInput, ModelOutput


class ModelWorker:
    def __init__(self, model, model_config, server_config):
        self.server_config = server_config
        # decode-only forwards replay one CUDA graph per batch-size bucket (reference:
        # tokainfer/utils.py:528-635) when `use_cudagraphs` is set
        runner_conf = RunnerConfig(page_size=server_config.page_size, max_total_tokens=server_config.kv_cache_num_tokens,
                                   max_running_requests=server_config.max_seqs_per_forward, seed=server_config.seed,
                                   use_cudagraph=bool(server_config.use_cudagraphs),
                                   cudagraph_additonal_batch_size=(1, 2, 4, 8),
                                   cudagraph_max_batch_size=min(512, server_config.max_seqs_per_forward))
        if server_config.kv_cache_num_tokens is None:
            model_config.memory_fraction_static = server_config.memory_fraction
        self.runner = ModelRunner(model, model_config, runner_conf)
        self.device = self.runner.device
        self._post_init()

    def _post_init(self):
        r = self.runner
        self.page_size = r.page_size
        self.num_blocks = r.kv_pool.num_pages
        self.max_seqs = r.req_pool.size - 1
        self.last_tokens = torch.zeros(r.req_pool.size, dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ lifecycle
    def initialize(self):
        if self.runner.kv_pool is None:
            self.runner.initialize()
            self._post_init()

    def cleanup(self):
        self.runner.cleanup()

    def load_state_dict(self, state_dict, assign=True):
        self.runner.load_state_dict(state_dict, assign=assign)

    @torch.no_grad()
    def update_weights_broadcast(self, src=0, group=None):
        import torch.distributed as dist

        for _, p in sorted(self.runner.model.named_parameters()):
            dist.broadcast(p.data, src=src, group=group)

    def handle(self, command: Command):
        if command.kind == "cleanup":
            self.cleanup()
        elif command.kind == "initialize":
            self.initialize()
        elif command.kind == "load_state_dict":
            self.load_state_dict(command.payload)
        else:
            raise ValueError(f"unknown command {command.kind}")

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def run(self, inp: ModelInput) -> ModelOutput:
        r, ps, dev = self.runner, self.page_size, self.device
        table = r.req_pool.req_to_pages
        for row, start, pages in inp.page_updates:
            # blocks are numbered from 0 by the manager; page 0 of the pool is the scratch page
            table[row, start:start + len(pages)] = torch.tensor([p + 1 for p in pages], dtype=torch.int32).to(dev)
        n_entries = len(inp.batch_indices)
        if n_entries == 0:
            return ModelOutput(inp.step_id, [], [], [])
        if all(t is None for t in inp.tokens):
            return self._run_decode(inp)
        lens = [1 if t is None else len(t) for t in inp.tokens]
        indptr = [0]
        for n in lens:
            indptr.append(indptr[-1] + n)
        total = indptr[-1]
        ids = torch.zeros(total, dtype=torch.int64)
        positions = torch.zeros(total, dtype=torch.int64)
        from_device_rows, from_device_pos = [], []
        for i, (toks, prefix, n) in enumerate(zip(inp.tokens, inp.prefix_lens, lens)):
            s = indptr[i]
            if toks is None:
                from_device_rows.append(inp.batch_indices[i])
                from_device_pos.append(s)
            else:
                ids[s:s + n] = torch.tensor(toks, dtype=torch.int64)
            positions[s:s + n] = torch.arange(prefix, prefix + n)
        ids, positions = ids.to(dev), positions.to(dev)
        if from_device_rows:
            ids[torch.tensor(from_device_pos, device=dev)] = self.last_tokens[torch.tensor(from_device_rows, device=dev)]
        rows = torch.tensor(inp.batch_indices, dtype=torch.int64, device=dev)
        entry_of_token = torch.repeat_interleave(torch.arange(n_entries, device=dev),
                                                 torch.tensor(lens, device=dev))
        page_of = table[rows[entry_of_token], (positions // ps)].to(torch.int64)
        out_loc = page_of * ps + positions % ps
        seq_lens = [p + n for p, n in zip(inp.prefix_lens, lens)]
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=dev)
        fb = ForwardBatch(
            mode=ForwardMode.EXTEND, input_ids=ids, positions=positions, out_cache_loc=out_loc,
            req_slots=i32(inp.batch_indices), seq_lens=i32(seq_lens), extend_lens=i32(lens),
            prefix_lens=i32(inp.prefix_lens), qo_indptr=i32(indptr), page_table=table, max_seq_len=max(seq_lens),
            max_extend_len=max(lens), page_size=ps,
            sample_indices=torch.tensor([x - 1 for x in indptr[1:]], dtype=torch.int64, device=dev),
            seq_lens_cpu=seq_lens, extend_lens_cpu=lens)
        logits = r.forward(fb)                                    # [entries, vocab]
        return self._sample(inp, logits, rows)

    def _sample(self, inp, logits, rows):
        r, dev = self.runner, self.device
        f32 = lambda xs: torch.tensor(xs, dtype=torch.float32, device=dev)
        sampling = BatchSamplingParams(
            temperatures=f32(inp.temperatures).view(-1, 1), top_ps=f32(inp.top_ps),
            top_ks=torch.tensor([min(k if k > 0 else 1 << 30, 1 << 30) for k in inp.top_ks], dtype=torch.int32, device=dev),
            min_ps=f32(inp.min_ps), is_all_greedy=all(0 < k <= 1 for k in inp.top_ks),
            need_min_p_sampling=any(p > 0 for p in inp.min_ps),
            need_top_k_top_p=any(p < 1.0 for p in inp.top_ps) or any(1 < k < (1 << 29) for k in inp.top_ks))
        tokens, logprobs = r.sampler(logits, sampling)
        keep = [i for i, s in enumerate(inp.sample) if s]
        if not keep:
            return ModelOutput(inp.step_id, [], [], [])
        k = torch.tensor(keep, device=dev)
        kept_tokens, kept_lps = tokens[k], logprobs[k].float()
        self.last_tokens[rows[k]] = kept_tokens
        return LazyModelOutput(inp.step_id, [inp.batch_indices[i] for i in keep], kept_tokens, kept_lps)

    @torch.no_grad()
    def _run_decode(self, inp: ModelInput):
        """Every entry is one decode token fed from the device-side buffer: the split-KV decode
        kernel path, no host-built token tensor."""
        r, ps, dev = self.runner, self.page_size, self.device
        table = r.req_pool.req_to_pages
        rows = torch.tensor(inp.batch_indices, dtype=torch.int64, device=dev)
        positions = torch.tensor(inp.prefix_lens, dtype=torch.int64, device=dev)
        page_of = table[rows, positions // ps].to(torch.int64)
        seq_lens = [p + 1 for p in inp.prefix_lens]
        fb = ForwardBatch(
            mode=ForwardMode.DECODE, input_ids=self.last_tokens[rows], positions=positions,
            out_cache_loc=page_of * ps + positions % ps,
            req_slots=torch.tensor(inp.batch_indices, dtype=torch.int32, device=dev),
            seq_lens=torch.tensor(seq_lens, dtype=torch.int32, device=dev), page_table=table,
            max_seq_len=max(seq_lens), max_extend_len=1, page_size=ps, seq_lens_cpu=seq_lens)
        return self._sample(inp, r.forward_decode(fb), rows)


class LazyModelOutput:
    """Result of a forward whose sampled tokens are still on their way to the host: the copy
    into pinned memory is enqueued behind the forward and only waited for when the manager reads
    the tokens, by which time later forwards are already queued on the device."""

    def __init__(self, step_id, batch_indices, tokens_dev, logprobs_dev):
        self.step_id, self.batch_indices = step_id, batch_indices
        pin = tokens_dev.is_cuda
        self._tok = torch.empty(tokens_dev.shape, dtype=tokens_dev.dtype, pin_memory=pin)
        self._lp = torch.empty(logprobs_dev.shape, dtype=logprobs_dev.dtype, pin_memory=pin)
        self._tok.copy_(tokens_dev, non_blocking=True)
        self._lp.copy_(logprobs_dev, non_blocking=True)
        self._event = None
        if pin:
            self._event = torch.cuda.Event()
            self._event.record()
        self._done = None

    def materialize(self):
        if self._done is None:
            if self._event is not None:
                self._event.synchronize()
            self._done = ModelOutput(self.step_id, self.batch_indices, self._tok.tolist(), self._lp.tolist())
        return self._done

    @property
    def tokens(self):
        return self.materialize().tokens

    @property
    def logprobs(self):
        return self.materialize().logprobs


def worker_main(build_model, model_config, server_config, in_q, out_q):
    """Entry point of the worker process: build the model, then serve inputs until shutdown."""
    model = build_model()
    worker = ModelWorker(model, model_config, server_config)
    out_q.put(("ready", worker.num_blocks, worker.max_seqs))
    while True:
        msg = in_q.get()
        if isinstance(msg, Command):
            if msg.kind == "shutdown":
                break
            worker.handle(msg)
            out_q.put(("done", msg.kind))
            if msg.kind == "initialize":
                out_q.put(("ready", worker.num_blocks, worker.max_seqs))
            continue
        out = worker.run(msg)
        out_q.put(out.materialize() if hasattr(out, "materialize") else out)
