"""Owns the model, the KV / request pools and the forward paths of the engine (reference:
infer/engine/model_runner.py:14-252).

Decode runs `n` steps ahead of the host: sampled tokens, positions, sequence lengths and KV
slots are advanced on the device between steps (the page table already holds the pages those
steps will open), so the host reads tokens once per `n` steps instead of once per token.
With `use_cudagraph` each step replays a captured graph of the model forward for the batch
bucket.
"""

from __future__ import annotations

import torch

from halite_b200.infer.batch import ForwardBatch, ForwardMode
from halite_b200.infer.memory_pool import PagedKVPool, RequestToPagePool
from halite_b200.infer.sampler import Sampler
from halite_b200.infer.types import ModelConfig, ServerConfig
from halite_b200.utils import get_torch_dtype


def get_gpu_memory(device, gpu_id=0, distributed=False):
    """(available, total) GiB on the device; with `distributed` the minimum over ranks."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return 4.0, 4.0
    free, total = torch.cuda.mem_get_info(gpu_id if dev.index is None else dev.index)
    t = torch.tensor([free / 2 ** 30, total / 2 ** 30], dtype=torch.float32, device=dev)
    if distributed and torch.distributed.is_initialized():
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
    return float(t[0]), float(t[1])


class ModelRunner:
    def __init__(self, model, model_config: ModelConfig, server_config: ServerConfig):
        self.model = model
        self.model_config = model_config
        self.server_config = server_config
        self.sampler = Sampler(seed=server_config.seed)
        self.device = torch.device(model_config.device)
        if self.device.type == "cuda" and self.device.index is None:
            # "cuda" without an index: `gpu_id` when it names a device, else the process's current one
            self.device = torch.device("cuda", model_config.gpu_id or torch.cuda.current_device())
        self.page_size = server_config.page_size
        dtype = model_config.kv_cache_dtype
        if dtype == "auto":
            # the model is usually still on the meta device here: bf16 on a GPU, fp32 on CPU
            first = next((p for p in model.parameters() if p.is_floating_point()), None)
            if first is not None and not first.is_meta:
                dtype = first.dtype
            else:
                dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.kv_cache_dtype = get_torch_dtype(dtype)
        self.req_pool = None
        self.kv_pool = None
        self.graphs = {}
        self.graph_state = None
        self.workspace = None
        self._resharder = None
        self._resharder_src = None
        self.initialize()

    # ------------------------------------------------------------------ lifecycle
    def estimate_max_tokens(self):
        mc = self.model_config
        if self.server_config.max_total_tokens is not None:
            return int(self.server_config.max_total_tokens)
        avail, total = get_gpu_memory(self.device, mc.gpu_id, mc.distributed)
        cell = (mc.n_key_value_heads // mc.tp_size if mc.n_key_value_heads >= mc.tp_size else 1) \
            * mc.head_dim * mc.n_layers * 2 * torch.empty(0, dtype=self.kv_cache_dtype).element_size()
        rest = avail - total * (1 - mc.memory_fraction_static)
        n = int(rest * (1 << 30) // cell)
        if n <= 0:
            raise RuntimeError("not enough device memory for a KV cache: raise memory_fraction_static")
        return n

    def initialize(self):
        mc, sc = self.model_config, self.server_config
        self.max_total_tokens = self.estimate_max_tokens() // self.page_size * self.page_size
        n_pages = self.max_total_tokens // self.page_size
        self.max_running_requests = min(sc.max_running_requests, max(self.max_total_tokens // 2, 1))
        self.max_requests = min(max(int(self.max_total_tokens / mc.context_len * 512), 2048), 4096)
        max_pages_per_req = (mc.context_len + 4 + self.page_size - 1) // self.page_size
        # one extra, never allocated row: padded CUDA-graph entries point at it (all page 0)
        self.req_pool = RequestToPagePool(self.max_requests + 1, max_pages_per_req, self.device)
        self.req_pool.free_slots = list(range(self.max_requests))
        self.pad_slot = self.max_requests
        kv_heads = max(mc.n_key_value_heads // mc.tp_size, 1)
        self.kv_pool = PagedKVPool(n_pages, self.page_size, mc.n_layers, kv_heads, mc.head_dim,
                                   self.kv_cache_dtype, self.device)
        if hasattr(self.model, "set_kv_pool"):
            self.model.set_kv_pool(self.kv_pool)
        self.graphs = {}
        self.graph_state = None
        if self.device.type == "cuda":
            q_heads = max(mc.n_heads // mc.tp_size, 1)
            self.workspace = torch.empty(self.decode_workspace_numel(q_heads, mc.head_dim),
                                         dtype=torch.float32, device=self.device)

    def decode_workspace_numel(self, q_heads, head_dim, max_batch=None, max_splits=32):
        b = max_batch or min(self.max_running_requests, 4096)
        return b * q_heads * max_splits * (head_dim + 2)

    def reset_pools(self):
        """Forget every request and page (pools and graphs stay where they are)."""
        self.kv_pool.clear()
        self.req_pool.clear()
        self.req_pool.free_slots = list(range(self.max_requests))

    def cleanup(self):
        """Give the device memory back (weights and pools) so training can use it."""
        self.model.to("meta")
        self._resharder = None                 # its destination tensors are gone with the weights
        if hasattr(self.model, "set_kv_pool"):
            self.model.set_kv_pool(None)       # the attention layers hold the pool too
        self.req_pool = None
        self.kv_pool = None
        self.graphs = {}
        self.graph_state = None
        self.workspace = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def load_state_dict(self, state_dict, assign=True):
        from halite_b200.distributed.state_dict import reshard_state_dict

        tp = getattr(self.model, "_infer_tp", None)
        tp_kw = {} if tp is None else dict(tp_rank=tp.rank, tp_size=tp.size, tp_plan=self.model._infer_tp_plan)
        resident = self.server_config.keep_resident and not any(p.is_meta for p in self.model.parameters())
        if resident:
            # same storage, new values: captured graphs and tensor maps stay valid
            reshard_state_dict(state_dict, self.model.state_dict(), device=self.device, in_place=True, **tp_kw)
            return
        self.model.to("meta")
        target = self.model.state_dict()
        sd = reshard_state_dict(state_dict, target, device=self.device, **tp_kw)
        if not assign:
            self.model.to_empty(device=self.device)
        self.model.load_state_dict(sd, assign=assign)
        if hasattr(self.model, "init_buffers"):
            self.model.init_buffers(self.device)
        if hasattr(self.model, "set_kv_pool") and self.kv_pool is not None:
            self.model.set_kv_pool(self.kv_pool)
        self.graphs = {}

    def load_from_model(self, train_model):
        """Take the weights of a sharded training model with the one-launch reshard kernel
        (`parallel/reshard.py`): the engine's tensors are allocated once in its own layout (this
        rank's tensor-parallel slices) and filled straight from the flat unit buffers, or from the
        ranks' shards over NVLink when the trainer keeps only shards. Falls back to
        `load_state_dict(train_model.state_dict())` off the GPU or for an unsharded model."""
        if self.device.type != "cuda" or getattr(train_model, "_hb_fsdp", None) is None:
            return self.load_state_dict(train_model.state_dict())
        from halite_b200.parallel.reshard import FusedResharder

        tp = getattr(self.model, "_infer_tp", None)
        if any(p.is_meta for p in self.model.parameters()) or self._resharder is None \
                or self._resharder_src is not train_model:
            self.model.to("meta")
            target = {k: torch.empty(v.shape, dtype=next(iter(train_model._hb_fsdp.units)).param_dtype,
                                     device=self.device)
                      for k, v in self.model.state_dict().items()}
            self.model.load_state_dict(target, assign=True)
            if hasattr(self.model, "init_buffers"):
                self.model.init_buffers(self.device)
            if hasattr(self.model, "set_kv_pool") and self.kv_pool is not None:
                self.model.set_kv_pool(self.kv_pool)
            self.graphs = {}
            # after packing, q | k | v (gate | up) are views of one matrix: the state dict still
            # names them separately and every view is contiguous, which is all the kernel needs
            live = dict(self.model.state_dict())
            self._resharder = FusedResharder(train_model, live, tp.rank if tp else 0, tp.size if tp else 1,
                                             getattr(self.model, "_infer_tp_plan", None))
            self._resharder_src = train_model
        self._resharder.run()

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, fb: ForwardBatch):
        fb.workspace = self.workspace
        return self.model(fb)

    @torch.no_grad()
    def forward_decode(self, fb: ForwardBatch):
        """One decode forward: replays the captured graph of the batch's size bucket when CUDA
        graphs are on (capturing it at first use), else runs eagerly."""
        graph = self._graph_for(fb.batch_size) if self.server_config.use_cudagraph else None
        if graph is not None:
            return self._replay(graph, fb)
        return self.forward(fb)

    @torch.no_grad()
    def forward_and_sample(self, batch):
        logits = self.forward(batch.forward_batch)
        ids, logprobs = self.sampler(logits, batch.sampling)
        return logits, ids, logprobs

    @torch.no_grad()
    def decode_steps(self, batch, n_steps, last_tokens=None):
        """Run `n_steps` decode steps without a host round trip. The batch has already had
        `alloc_for_decode(n_steps)` applied. Returns (ids [n, B], logprobs [n, B]) on device."""
        fb = batch.prepare_for_decode(last_tokens)
        ps = self.page_size
        B = fb.batch_size
        all_ids, all_lp = [], []
        slots64 = fb.req_slots.long()
        graph = self._graph_for(B) if self.server_config.use_cudagraph else None
        for s in range(n_steps):
            if graph is not None:
                logits = self._replay(graph, fb)
            else:
                logits = self.forward(fb)
            ids, lp = self.sampler(logits, batch.sampling)
            all_ids.append(ids)
            all_lp.append(lp)
            if s + 1 < n_steps:
                positions = fb.positions + 1
                pages = fb.page_table[slots64, positions // ps].long()
                fb = ForwardBatch(
                    mode=ForwardMode.DECODE, input_ids=ids, positions=positions,
                    out_cache_loc=pages * ps + positions % ps, req_slots=fb.req_slots,
                    seq_lens=fb.seq_lens + 1, page_table=fb.page_table, max_seq_len=fb.max_seq_len + 1,
                    max_extend_len=1, page_size=ps,
                    seq_lens_cpu=[x + 1 for x in fb.seq_lens_cpu] if fb.seq_lens_cpu else None)
        for r in batch.requests:
            r.pending_tokens += n_steps
        return torch.stack(all_ids), torch.stack(all_lp)

    # ------------------------------------------------------------------ CUDA graphs
    def graph_sizes(self):
        sc = self.server_config
        sizes = set(sc.cudagraph_additonal_batch_size) | set(
            range(sc.cudagraph_step, sc.cudagraph_max_batch_size + 1, sc.cudagraph_step))
        return sorted(s for s in sizes if s > 0)

    def _graph_capturable(self):
        """A decode forward can be captured only when every attention layer runs the paged kernels: the
        plain-PyTorch path they fall back to (other head sizes or cache types, soft-cap, windows) reads
        lengths on the host."""
        if getattr(self, "_capturable", None) is None:
            mc = self.model_config
            ok = self.kv_cache_dtype == torch.bfloat16 and mc.head_dim in (64, 128)
            for m in self.model.modules():
                if getattr(m, "softcap", 0.0) or getattr(m, "window_size", None) is not None:
                    ok = False
            first = next((p for p in self.model.parameters() if p.is_floating_point()), None)
            if first is not None and first.dtype != torch.bfloat16:
                ok = False
            self._capturable = ok
        return self._capturable

    def _graph_for(self, batch_size):
        if self.device.type != "cuda" or not self._graph_capturable():
            return None
        sizes = self.graph_sizes()
        bucket = next((s for s in sizes if s >= batch_size), None)
        if bucket is None:
            return None
        if bucket not in self.graphs:
            self.graphs[bucket] = self._capture(bucket)
        return self.graphs[bucket]

    def _static_batch(self, bucket):
        dev = self.device
        fb = ForwardBatch(
            mode=ForwardMode.DECODE,
            input_ids=torch.zeros(bucket, dtype=torch.int64, device=dev),
            positions=torch.zeros(bucket, dtype=torch.int64, device=dev),
            out_cache_loc=torch.zeros(bucket, dtype=torch.int64, device=dev),
            req_slots=torch.full((bucket,), self.pad_slot, dtype=torch.int32, device=dev),
            seq_lens=torch.ones(bucket, dtype=torch.int32, device=dev),
            page_table=self.req_pool.req_to_pages, max_seq_len=self.model_config.context_len,
            max_extend_len=1, page_size=self.page_size)
        fb.workspace = self.workspace
        return fb

    def _capture(self, bucket):
        fb = self._static_batch(bucket)
        # warm up on a side stream (allocator, lazy init), then capture
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self.model(fb)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.model(fb)
        return {"graph": g, "fb": fb, "out": out, "bucket": bucket}

    def _replay(self, graph, fb):
        st = graph["fb"]
        B = fb.batch_size
        st.input_ids[:B].copy_(fb.input_ids)
        st.positions[:B].copy_(fb.positions)
        st.out_cache_loc[:B].copy_(fb.out_cache_loc)
        st.req_slots[:B].copy_(fb.req_slots)
        st.seq_lens[:B].copy_(fb.seq_lens)
        if B < graph["bucket"]:
            st.req_slots[B:].fill_(self.pad_slot)
            st.seq_lens[B:].fill_(1)
            st.positions[B:].zero_()
            st.out_cache_loc[B:].zero_()
        graph["graph"].replay()
        return graph["out"][:B]
