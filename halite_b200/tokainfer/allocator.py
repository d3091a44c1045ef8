"""Block (page) allocator with a page-granular prefix tree
(reference: tokainfer/engine/allocator.py:11-445).

Every KV page is a `PrefixTreeBlock`. A block is either *floating* (owned by one sequence, or
free) or *in the tree*: keyed by its 16 token ids under the block holding the previous 16, so a
chain from the root spells a prefix. Tree blocks carry the set of sequences using them; a tree
leaf used by nobody can be recycled (least recently used first). A new sequence walks the tree to
reuse the longest cached prefix, but never the page that would contain its last prompt token: that
token must be computed to produce the first logits.
"""

from __future__ import annotations

import itertools


class NoSpaceException(ValueError):
    pass


class PrefixTreeBlock:
    __slots__ = ("idx", "parent", "children", "contents", "seq_ids", "last_used", "in_tree")

    def __init__(self, idx):
        self.idx = idx
        self.wipe()

    def wipe(self):
        self.parent = None
        self.children = {}
        self.contents = None          # tuple of page_size token ids once in the tree
        self.seq_ids = set()
        self.last_used = 0
        self.in_tree = False

    def is_root(self):
        return self.idx < 0

    def __lt__(self, other):
        return self.last_used < other.last_used

    def __repr__(self):
        return f"Block({self.idx}, users={len(self.seq_ids)}, tree={self.in_tree})"


def truncate_to_multiple(xs, multiple):
    return xs[: len(xs) // multiple * multiple]


class BlockAllocator:
    def __init__(self, num_blocks: int, page_size: int):
        self.num_blocks, self.page_size = num_blocks, page_size
        self.initialize()

    def initialize(self):
        self.blocks = [PrefixTreeBlock(i) for i in range(self.num_blocks)]
        self.root = PrefixTreeBlock(-1)
        self.root.in_tree = True
        self.free_floating = list(range(self.num_blocks - 1, -1, -1))    # stack of never/no-longer used ids
        self._clock = itertools.count(1)

    def cleanup(self):
        self.blocks, self.root, self.free_floating = [], None, []

    # ------------------------------------------------------------------ accounting
    def _evictable_leaves(self):
        out, stack = [], [self.root]
        while stack:
            b = stack.pop()
            if b.children:
                stack.extend(b.children.values())
            elif not b.is_root() and not b.seq_ids:
                out.append(b)
        return out

    def num_free_blocks(self):
        """Blocks obtainable right now: unused floating blocks + unused tree blocks (a chain of
        unused tree blocks becomes evictable leaf by leaf)."""
        n, stack = len(self.free_floating), [self.root]
        while stack:
            b = stack.pop()
            for c in b.children.values():
                if not c.seq_ids:
                    n += self._subtree_unused(c)
                else:
                    stack.append(c)
        return n

    def _subtree_unused(self, b):
        # a subtree is fully reclaimable iff nobody uses any block in it; users of a child always
        # use the parent too, so checking the top block suffices
        n, stack = 0, [b]
        while stack:
            x = stack.pop()
            n += 1
            stack.extend(x.children.values())
        return n

    def num_used_blocks(self):
        return self.num_blocks - self.num_free_blocks()

    def fraction_used(self):
        return self.num_used_blocks() / max(self.num_blocks, 1)

    # ------------------------------------------------------------------ prefix tree
    def prefix_match(self, input_ids):
        """Blocks of the longest cached prefix (whole pages)."""
        ps, node, out = self.page_size, self.root, []
        for start in range(0, len(input_ids) - ps + 1, ps):
            child = node.children.get(tuple(input_ids[start:start + ps]))
            if child is None:
                break
            out.append(child)
            node = child
        return out

    def _take_block(self):
        if self.free_floating:
            return self.blocks[self.free_floating.pop()]
        leaves = self._evictable_leaves()
        if not leaves:
            raise NoSpaceException("no free KV blocks")
        victim = min(leaves)
        del victim.parent.children[victim.contents]
        victim.wipe()
        return victim

    def allocate_with_prefix_match(self, seq_id, input_ids):
        """(cached block ids, new block ids) covering the whole prompt. Raises NoSpaceException
        (leaving nothing allocated) when the pool cannot hold it."""
        ps = self.page_size
        usable = (len(input_ids) - 1) // ps * ps              # never the page of the last prompt token
        cached = self.prefix_match(input_ids[:usable])
        need = -(-len(input_ids) // ps) - len(cached)
        now = next(self._clock)
        for b in cached:                                      # pin before evicting anything
            b.seq_ids.add(seq_id)
            b.last_used = now
        if need > self.num_free_blocks():
            for b in cached:
                b.seq_ids.discard(seq_id)
            raise NoSpaceException(f"need {need} blocks, {self.num_free_blocks()} available")
        fresh = []
        for _ in range(need):
            b = self._take_block()
            b.seq_ids.add(seq_id)
            b.last_used = now
            fresh.append(b)
        return [b.idx for b in cached], [b.idx for b in fresh]

    def num_blocks_needed(self, kv_indices, length):
        return max(0, -(-length // self.page_size) - len(kv_indices))

    def allocate_up_to_length(self, seq_id, kv_indices, length):
        """Grow a sequence's block list to cover `length` tokens; returns the new block ids."""
        need = self.num_blocks_needed(kv_indices, length)
        if need > self.num_free_blocks():
            raise NoSpaceException(f"need {need} blocks, {self.num_free_blocks()} available")
        now, out = next(self._clock), []
        for _ in range(need):
            b = self._take_block()
            b.seq_ids.add(seq_id)
            b.last_used = now
            out.append(b.idx)
        return out

    def free_and_update(self, seq_id, kv_indices, token_ids):
        """Release a sequence. Its full pages whose KV was written (`token_ids` = tokens in the
        cache) join the prefix tree for later reuse; duplicates of pages already in the tree and
        the partial last page go back to the free list."""
        ps, node = self.page_size, self.root
        now = next(self._clock)
        n_full = len(token_ids) // ps
        for i, idx in enumerate(kv_indices):
            b = self.blocks[idx]
            b.seq_ids.discard(seq_id)
            if i < n_full and node is not None:
                key = tuple(token_ids[i * ps:(i + 1) * ps])
                existing = node.children.get(key)
                if existing is b:
                    node = b
                elif existing is not None:
                    existing.last_used = now
                    if not b.in_tree and not b.seq_ids:
                        b.wipe()
                        self.free_floating.append(b.idx)
                    node = existing
                elif not b.in_tree:
                    b.parent, b.contents, b.in_tree, b.last_used = node, key, True, now
                    node.children[key] = b
                    node = b
                else:
                    node = None            # already elsewhere in the tree: stop extending the chain
            elif not b.in_tree and not b.seq_ids:
                b.wipe()
                self.free_floating.append(b.idx)

    # ------------------------------------------------------------------ checks
    def sanity_checks(self, seq_ids=None):
        seen = set(self.free_floating)
        assert len(seen) == len(self.free_floating), "duplicate ids in the free list"
        stack = [self.root]
        while stack:
            b = stack.pop()
            for key, c in b.children.items():
                assert c.parent is b and c.contents == key and c.in_tree and len(key) == self.page_size
                assert c.idx not in seen, f"block {c.idx} is both free and in the tree"
                assert c.seq_ids <= b.seq_ids or b.is_root(), "a child is used by a sequence its parent is not"
                seen.add(c.idx)
                stack.append(c)
        for b in self.blocks:
            if not b.in_tree and b.idx not in seen:
                assert b.seq_ids, f"block {b.idx} is neither free, in the tree, nor owned"
            if seq_ids is not None:
                assert b.seq_ids <= seq_ids, f"block {b.idx} held by unknown sequences"
            if b.idx in self.free_floating:
                assert not b.seq_ids


class BatchIndexAllocator:
    """Rows of the worker's page table."""

    def __init__(self, max_indices: int):
        self.max_indices = max_indices
        self.initialize()

    def initialize(self):
        self.free = list(range(self.max_indices - 1, -1, -1))

    def cleanup(self):
        self.free = []

    def allocate(self):
        if not self.free:
            raise NoSpaceException("no free batch index")
        return self.free.pop()

    def free_index(self, idx):
        self.free.append(idx)

    def available(self):
        return len(self.free)
