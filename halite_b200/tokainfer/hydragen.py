"""Shared-prefix grouping of decoding sequences (reference: tokainfer/engine/hydragen.py:13-207).

Sequences whose KV page lists start with the same pages share that prefix's keys and values.
`group_for_hydragen` finds groups of at least `min_group_size` sequences sharing at least
`min_prefix_len` tokens, so attention over the shared part can be computed once per group (as a
dense, non-causal block over the group's queries) and merged with each sequence's own suffix by
the usual log-sum-exp combine. `reorder_decoding_seqs_for_hydragen` makes group members
contiguous in the batch.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class HydragenGroup:
    block_ids: list          # shared pages, in order
    seq_ids: list            # members


def group_for_hydragen(seqs, page_size, min_group_size, min_prefix_len):
    """Greedy trie walk over page-id lists. Returns (groups, ungrouped sequence ids); a sequence
    belongs to at most one group (its deepest qualifying prefix)."""
    min_pages = -(-min_prefix_len // page_size)
    trie = {}
    for s in seqs:
        node = trie
        # the page holding the newest token is still being written: exclude it
        usable = s.kv_indices[: max(0, (s.total_scheduled_len() - 1) // page_size)]
        for page in usable:
            node = node.setdefault(page, {"#": []})
            node["#"].append(s.id)
    groups, taken = [], set()

    def walk(node, path):
        # deepest first, so members join the longest shared prefix available to them
        for page, child in node.items():
            if page == "#":
                continue
            walk(child, path + [page])
        members = [i for i in node.get("#", []) if i not in taken]
        if len(path) >= min_pages and len(members) >= min_group_size:
            groups.append(HydragenGroup(list(path), members))
            taken.update(members)

    walk(trie, [])
    ungrouped = [s.id for s in seqs if s.id not in taken]
    return groups, ungrouped


def restrict_hydragen_groups(groups, max_groups):
    """Keep the groups that save the most work (members x shared pages)."""
    ranked = sorted(groups, key=lambda g: len(g.seq_ids) * len(g.block_ids), reverse=True)
    return ranked[:max_groups], [i for g in ranked[max_groups:] for i in g.seq_ids]


def reorder_decoding_seqs_for_hydragen(seqs, groups):
    by_id = {s.id: s for s in seqs}
    ordered, seen = [], set()
    for g in groups:
        for i in g.seq_ids:
            ordered.append(by_id[i])
            seen.add(i)
    ordered.extend(s for s in seqs if s.id not in seen)
    return ordered
