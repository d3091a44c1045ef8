"""Device memory pools of the engine (reference: infer/engine/memory_pool.py:4-158), paged.

`PagedKVPool` holds per layer one K and one V tensor of shape [pages, page_size, kv_heads,
head_dim]. Page 0 is a scratch page: padded CUDA-graph rows write there. A token's flat
slot is `page * page_size + offset`. `RequestToPagePool` maps a request slot to its page ids.
Free lists live on the host.
"""

from __future__ import annotations

import torch


class RequestToPagePool:
    def __init__(self, max_requests: int, max_pages_per_request: int, device):
        self.size = max_requests
        self.max_pages = max_pages_per_request
        self.device = device
        self.req_to_pages = torch.zeros(max_requests, max_pages_per_request, dtype=torch.int32, device=device)
        self.free_slots = list(range(max_requests))

    def available_size(self):
        return len(self.free_slots)

    def alloc(self, n: int):
        if n > len(self.free_slots):
            return None
        out, self.free_slots = self.free_slots[:n], self.free_slots[n:]
        return out

    def free(self, slots):
        if isinstance(slots, int):
            slots = [slots]
        self.free_slots.extend(slots)

    def write(self, slot: int, start_page: int, page_ids):
        if len(page_ids) == 0:
            return
        t = torch.as_tensor(page_ids, dtype=torch.int32)
        self.req_to_pages[slot, start_page:start_page + len(page_ids)] = t.to(self.device, non_blocking=True)

    def clear(self):
        self.free_slots = list(range(self.size))


class PagedKVPool:
    def __init__(self, num_pages: int, page_size: int, n_layers: int, kv_heads: int, head_dim: int,
                 dtype, device):
        self.num_pages = num_pages
        self.page_size = page_size
        self.n_layers = n_layers
        self.kv_heads = kv_heads
        self.head_dim = head_dim
        self.dtype = dtype
        self.device = device
        # +1: page 0 is never handed out
        shape = (num_pages + 1, page_size, kv_heads, head_dim)
        self.k_buffer = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.v_buffer = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.free_pages = list(range(1, num_pages + 1))

    @property
    def size(self):
        """Capacity in tokens."""
        return self.num_pages * self.page_size

    def available_pages(self):
        return len(self.free_pages)

    def available_size(self):
        return len(self.free_pages) * self.page_size

    def alloc(self, n_pages: int):
        if n_pages > len(self.free_pages):
            return None
        out = self.free_pages[-n_pages:] if n_pages else []
        if n_pages:
            del self.free_pages[-n_pages:]
        return out

    def free(self, pages):
        self.free_pages.extend(pages)

    def clear(self):
        self.free_pages = list(range(1, self.num_pages + 1))

    def bytes_per_token(self):
        return 2 * self.n_layers * self.kv_heads * self.head_dim * torch.empty(0, dtype=self.dtype).element_size()

    def get_kv_buffer(self, layer_id):
        return self.k_buffer[layer_id], self.v_buffer[layer_id]
