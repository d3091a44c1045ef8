"""Page-granular radix tree over token prefixes (reference: infer/engine/radix_cache.py:8-321
for the lifecycle, tokainfer/engine/allocator.py:11-445 for page-sized keys).

Each node owns whole KV pages: its key is a token sequence whose length is a multiple of the
page size and its value is the list of page ids that hold those tokens. Requests that share a
prefix share the pages. Nodes referenced by a running request are locked; unlocked leaves are
evicted least-recently-used first when the pool runs dry.
"""

from __future__ import annotations

import heapq
import time


class TreeNode:
    __slots__ = ("children", "parent", "key", "value", "lock_ref", "last_access_time")

    def __init__(self):
        self.children = {}
        self.parent = None
        self.key = []        # tokens, len % page_size == 0
        self.value = []      # page ids, len == len(key) // page_size
        self.lock_ref = 0
        self.last_access_time = time.monotonic()

    def __lt__(self, other):
        return self.last_access_time < other.last_access_time


class RadixCache:
    def __init__(self, page_size: int, kv_pool, disable: bool = False):
        self.page_size = page_size
        self.kv_pool = kv_pool
        self.disable = disable
        self.reset()

    def reset(self):
        self.root = TreeNode()
        self.root.lock_ref = 1
        self.evictable_pages = 0
        self.protected_pages = 0

    # ------------------------------------------------------------------ lookup
    def _child_key(self, tokens, start):
        return tuple(tokens[start:start + self.page_size])

    def _match_pages(self, key, tokens, start):
        """Number of whole pages of `key` equal to tokens[start:]."""
        ps = self.page_size
        n = 0
        limit = min(len(key), (len(tokens) - start) // ps * ps)
        while n < limit and key[n:n + ps] == tokens[start + n:start + n + ps]:
            n += ps
        return n // ps

    def match_prefix(self, tokens):
        """Longest cached prefix in whole pages: (page ids, last node). Splits a node when the
        match ends inside it, so the returned node covers exactly the match."""
        if self.disable:
            return [], self.root
        tokens = list(tokens)
        node, pos, pages = self.root, 0, []
        now = time.monotonic()
        while len(tokens) - pos >= self.page_size:
            child = node.children.get(self._child_key(tokens, pos))
            if child is None:
                break
            child.last_access_time = now
            n = self._match_pages(child.key, tokens, pos)
            if n * self.page_size < len(child.key):
                child = self._split(child, n)
                pages.extend(child.value)
                node = child
                break
            pages.extend(child.value)
            pos += len(child.key)
            node = child
        return pages, node

    def _split(self, child, n_pages):
        """Split `child` after n_pages; returns the new upper node."""
        ps = self.page_size
        upper = TreeNode()
        upper.parent = child.parent
        upper.key = child.key[: n_pages * ps]
        upper.value = child.value[:n_pages]
        upper.lock_ref = child.lock_ref
        upper.last_access_time = child.last_access_time
        child.parent.children[tuple(upper.key[:ps])] = upper
        child.key = child.key[n_pages * ps:]
        child.value = child.value[n_pages:]
        child.parent = upper
        upper.children[tuple(child.key[:ps])] = child
        return upper

    # ------------------------------------------------------------------ insert
    def insert(self, tokens, pages):
        """Insert whole pages (len(tokens) == len(pages) * page_size). Returns the number of
        leading pages that were already cached (the caller frees its duplicates of those)."""
        if self.disable:
            return 0
        tokens = list(tokens)
        ps = self.page_size
        assert len(tokens) == len(pages) * ps
        node, pos, shared = self.root, 0, 0
        now = time.monotonic()
        while pos < len(tokens):
            child = node.children.get(self._child_key(tokens, pos))
            if child is None:
                new = TreeNode()
                new.parent = node
                new.key = tokens[pos:]
                new.value = list(pages[pos // ps:])
                new.last_access_time = now
                node.children[tuple(new.key[:ps])] = new
                self.evictable_pages += len(new.value)
                break
            child.last_access_time = now
            n = self._match_pages(child.key, tokens, pos)
            if n * ps < len(child.key):
                child = self._split(child, n)
            shared += n
            pos += n * ps
            node = child
        return shared

    # ------------------------------------------------------------------ locks
    def inc_lock_ref(self, node):
        if self.disable:
            return
        while node is not self.root and node is not None:
            if node.lock_ref == 0:
                self.evictable_pages -= len(node.value)
                self.protected_pages += len(node.value)
            node.lock_ref += 1
            node = node.parent

    def dec_lock_ref(self, node):
        if self.disable:
            return
        while node is not self.root and node is not None:
            if node.lock_ref == 1:
                self.evictable_pages += len(node.value)
                self.protected_pages -= len(node.value)
            node.lock_ref -= 1
            node = node.parent

    # ------------------------------------------------------------------ eviction
    def evictable_size(self):
        return self.evictable_pages * self.page_size

    def evict(self, n_pages: int):
        """Free at least n_pages from unlocked leaves (LRU first); returns pages freed."""
        if self.disable or n_pages <= 0:
            return 0
        leaves = [n for n in self._leaves() if n.lock_ref == 0]
        heapq.heapify(leaves)
        freed = 0
        while freed < n_pages and leaves:
            node = heapq.heappop(leaves)
            if node is self.root or node.lock_ref > 0:
                continue
            self.kv_pool.free(node.value)
            freed += len(node.value)
            self.evictable_pages -= len(node.value)
            parent = node.parent
            del parent.children[tuple(node.key[: self.page_size])]
            if not parent.children and parent is not self.root and parent.lock_ref == 0:
                heapq.heappush(leaves, parent)
        return freed

    def _leaves(self):
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            if not n.children:
                if n is not self.root:
                    out.append(n)
            else:
                stack.extend(n.children.values())
        return out

    # ------------------------------------------------------------------ request lifecycle
    def cache_finished_request(self, req, req_pool):
        """Keep the request's full pages in the tree, free the rest, release its lock."""
        ps = self.page_size
        pages = req.pages
        # the KV of the last generated token was never written
        n_tokens = len(req.input_ids) + max(len(req.output_ids) - 1, 0)
        n_full = min(n_tokens // ps, len(pages))
        if self.disable:
            self.kv_pool.free(pages)
        else:
            tokens = (list(req.input_ids) + list(req.output_ids))[: n_full * ps]
            shared = self.insert(tokens, pages[:n_full])
            # pages [n_prefix_pages, shared) duplicate what another request inserted meanwhile
            dup = pages[req.n_prefix_pages:shared]
            self.kv_pool.free(dup)
            self.kv_pool.free(pages[n_full:])
            self.dec_lock_ref(req.last_node)
        req_pool.free(req.req_slot)
        req.pages = []

    def cache_unfinished_request(self, req, req_pool):
        """After a prefill chunk: publish the full pages so far and re-point the request at the
        tree's copies (so a later duplicate insert cannot leave it on freed pages)."""
        if self.disable:
            return
        ps = self.page_size
        n_tokens = req.n_computed
        n_full = n_tokens // ps
        tokens = list(req.fill_ids[: n_full * ps])
        shared = self.insert(tokens, req.pages[:n_full])
        dup = req.pages[req.n_prefix_pages:shared]
        self.kv_pool.free(dup)
        new_pages, node = self.match_prefix(tokens)
        assert len(new_pages) == n_full
        req.pages[:n_full] = new_pages
        req_pool.write(req.req_slot, 0, new_pages)
        self.dec_lock_ref(req.last_node)
        self.inc_lock_ref(node)
        req.last_node = node
        req.n_prefix_pages = n_full

    def total_pages(self):
        n, stack = 0, [self.root]
        while stack:
            x = stack.pop()
            n += len(x.value)
            stack.extend(x.children.values())
        return n

    def sanity_check(self):
        """Invariants used by tests: page-aligned keys, counters equal a fresh walk."""
        ev = pr = 0
        stack = [self.root]
        while stack:
            x = stack.pop()
            for key, c in x.children.items():
                assert c.parent is x and tuple(c.key[: self.page_size]) == key
                assert len(c.key) == len(c.value) * self.page_size and len(c.value) > 0
                assert c.lock_ref >= 0
                if c.lock_ref == 0:
                    ev += len(c.value)
                else:
                    pr += len(c.value)
                    assert x is self.root or x.lock_ref >= c.lock_ref
                stack.append(c)
        assert ev == self.evictable_pages and pr == self.protected_pages, (ev, pr, self.evictable_pages, self.protected_pages)


class NativeRadixCache(RadixCache):
    """Same contract as `RadixCache`, with the tree itself in C++ (`_C.RadixTree`): matching,
    insertion, lock counting and LRU eviction run without touching Python objects per node. Node
    handles are integers (0 = root)."""

    def __init__(self, page_size: int, kv_pool, disable: bool = False):
        from halite_b200.csrc import build

        self._ext = build.load()
        self.page_size = page_size
        self.kv_pool = kv_pool
        self.disable = disable
        self.tree = self._ext.RadixTree(page_size)
        self.root = 0

    def reset(self):
        self.tree.reset()

    @property
    def evictable_pages(self):
        return self.tree.evictable_pages

    @property
    def protected_pages(self):
        return self.tree.protected_pages

    def match_prefix(self, tokens):
        if self.disable:
            return [], 0
        return self.tree.match_prefix(list(tokens))

    def insert(self, tokens, pages):
        if self.disable:
            return 0
        return self.tree.insert(list(tokens), list(pages))

    def inc_lock_ref(self, node):
        if not self.disable and node:
            self.tree.inc_lock_ref(node)

    def dec_lock_ref(self, node):
        if not self.disable and node:
            self.tree.dec_lock_ref(node)

    def evict(self, n_pages: int):
        if self.disable or n_pages <= 0:
            return 0
        freed = self.tree.evict(n_pages)
        self.kv_pool.free(freed)
        return len(freed)

    def total_pages(self):
        return self.tree.total_pages()

    def sanity_check(self):
        self.tree.sanity_check()


def make_radix_cache(page_size, kv_pool, disable=False, backend="auto"):
    """`backend`: "native" (C++ tree), "python", or "auto" = native when the extension is
    already built, else Python."""
    if backend == "python":
        return RadixCache(page_size, kv_pool, disable)
    if backend == "native":
        return NativeRadixCache(page_size, kv_pool, disable)
    try:
        from halite_b200.csrc import build

        if build.is_current():
            return NativeRadixCache(page_size, kv_pool, disable)
    except Exception:  # noqa: BLE001
        pass
    return RadixCache(page_size, kv_pool, disable)
