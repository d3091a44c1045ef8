"""Dataset helpers for generation-based evaluation (reference: projects/eval/dataset.py)."""

from __future__ import annotations

import json


def hf_dataset(path, name=None, split="test"):
    from datasets import load_dataset

    return load_dataset(path, name, split=split)


def jsonl_dataset(path):
    """A list of dict records from a local JSON-lines file (offline stand-in for `hf_dataset`)."""
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def first_n(dataset, n):
    """Few-shot sampler that always returns the first `n` examples as a list of dicts."""
    def sample():
        head = dataset[:n]
        if isinstance(head, dict):          # HF datasets slice into a dict of columns
            keys = list(head)
            return [{k: head[k][i] for k in keys} for i in range(len(head[keys[0]]))]
        return list(head)

    return sample
