"""KV caches for the dense (non-paged) generation loop (reference: transformers/cache_manager.py:4-185).

Layout here is `[batch, length, heads, head_dim]` (the layout the attention modules use), so the
length dimension is 1. `AttentionCache` grows by concatenation; `AllocatedCacheManager` owns
fixed buffers per layer and hands out `AllocatedCache` views that append in place, so a decode
loop allocates nothing per step.
"""

from __future__ import annotations

import torch

LENGTH_DIM = 1


class AttentionCache:
    def __init__(self, key, value, length_dim=LENGTH_DIM):
        self.key, self.value = key, value
        self.length_dim = length_dim
        self.length = key.shape[length_dim]

    def __getitem__(self, index):
        return (self.key, self.value)[index]

    def get(self, key, value):
        """Append the new keys / values and return everything cached so far."""
        return torch.cat((self.key, key), self.length_dim), torch.cat((self.value, value), self.length_dim)


class BasicCacheManager:
    def __init__(self, n_caches, length_dim=LENGTH_DIM):
        self.n_caches = n_caches
        self.length_dim = length_dim
        self.caches = [None] * n_caches

    def __len__(self):
        return self.n_caches

    def __getitem__(self, index):
        return self.get_cache(index)

    def get_cache(self, index, **kwargs):
        return self.caches[index]

    def update(self, index, cache):
        self.caches[index] = AttentionCache(*cache, length_dim=self.length_dim)

    def select(self, index):
        """Keep only the batch rows in `index` (finished sequences dropped)."""
        for i, c in enumerate(self.caches):
            if c is not None:
                self.caches[i] = AttentionCache(c.key[index], c.value[index], self.length_dim)


class AllocatedCache:
    def __init__(self, key, value, length):
        self.key, self.value, self.length = key, value, length

    def __getitem__(self, index):
        return (self.key[:, :self.length], self.value[:, :self.length])[index]

    def get(self, key, value):
        b, n = key.shape[0], key.shape[LENGTH_DIM]
        end = self.length + n
        self.key[:b, self.length:end] = key
        self.value[:b, self.length:end] = value
        self.length = end
        return self.key[:b, :end], self.value[:b, :end]


class AllocatedCacheManager:
    def __init__(self, n_cache, max_batch_size, max_length, n_head, head_dim, dtype=torch.float32,
                 device="cuda", caches=None):
        self.n_cache = n_cache
        self.lengths = [0] * n_cache
        self.max_batch_size, self.max_length = max_batch_size, max_length
        self.n_head, self.head_dim = n_head, head_dim
        self.dtype, self.device = dtype, device
        if caches is None:
            shape = (max_batch_size, max_length, n_head, head_dim)
            caches = [(torch.empty(shape, dtype=dtype, device=device), torch.empty(shape, dtype=dtype, device=device))
                      for _ in range(n_cache)]
        self.caches = caches

    def __len__(self):
        return self.n_cache

    def reset(self):
        self.lengths = [0] * self.n_cache

    def get_view(self, batch_size, batch_start=0, start_length=0):
        rows = slice(batch_start, batch_start + batch_size)
        views = [(k[rows, start_length:], v[rows, start_length:]) for k, v in self.caches]
        out = AllocatedCacheManager(self.n_cache, self.max_batch_size, self.max_length, self.n_head, self.head_dim,
                                    self.dtype, self.device, caches=views)
        out.lengths = [start_length] * self.n_cache
        return out

    def select(self, index):
        n = index.shape[0]
        for k, v in self.caches:
            k[:n] = k[index]
            v[:n] = v[index]

    def to(self, *args, **kwargs):
        self.caches = [(k.to(*args, **kwargs), v.to(*args, **kwargs)) for k, v in self.caches]
        return self

    def __getitem__(self, index):
        k, v = self.caches[index]
        return AllocatedCache(k, v, self.lengths[index])

    def shift(self, size):
        """Drop the oldest `size` positions (sliding window)."""
        length = self.lengths[0]
        for k, v in self.caches:
            k[:, :length - size] = k[:, size:length].clone()
            v[:, :length - size] = v[:, size:length].clone()
        self.lengths = [length - size] * self.n_cache

    def set_cache(self, caches, current_position, batch_start=0):
        for (ck, cv), (k, v) in zip(self.caches, caches):
            b, n = k.shape[0], k.shape[LENGTH_DIM]
            ck[batch_start:batch_start + b, current_position - n:current_position] = k
            cv[batch_start:batch_start + b, current_position - n:current_position] = v

    def update(self, index, cache):
        self.lengths[index] = cache[0].shape[LENGTH_DIM]
