"""Streaming preprocess operators (reference: data/preprocess.py:12-239). Each operator maps an
iterator of Records to an iterator of Records; stateful ones (`SequencePacking`) expose
`state_dict` / `load_state_dict` so a data loader can resume mid-stream."""

from __future__ import annotations

import json
from typing import Callable

import torch

from halite_b200.data.record import Record


class ReadRawText:
    def __init__(self, key="text"):
        self.key = key

    def __call__(self, iterator):
        for rec in iterator:
            rec[self.key] = rec.pop("data").decode("utf-8")
            yield rec


class ParseFeatures:
    """JSON payload -> record fields."""

    def __call__(self, iterator):
        for rec in iterator:
            payload = rec.pop("data")
            rec.update(json.loads(payload))
            yield rec


class SelectFeatures:
    def __init__(self, keys=("text",)):
        self.keys = keys

    def __call__(self, iterator):
        for rec in iterator:
            payload = rec.pop("data")
            for k in self.keys:
                rec[k] = payload[k]
            yield rec


class Map:
    def __init__(self, fn):
        self.fn = fn

    def __call__(self, iterator):
        for rec in iterator:
            rec.update(self.fn(rec))
            yield rec


class ApplyTemplate:
    def __init__(self, key, template):
        from halite_b200.projects.common.template import get_render_fn

        self.key = key
        self.template = get_render_fn(template)

    def __call__(self, iterator):
        for rec in iterator:
            rec[self.key] = self.template(rec)
            yield rec


class ApplyFormat:
    def __init__(self, key, format):
        self.key, self.format = key, format

    def __call__(self, iterator):
        for rec in iterator:
            rec[self.key] = self.format.format(**rec)
            yield rec


class Tokenize:
    def __init__(self, tokenizer, keys=("text",), output_keys=None, **tokenizer_kwargs):
        if output_keys is not None and len(output_keys) != len(keys):
            raise ValueError("output_keys must pair up with keys")
        self.tokenizer, self.keys, self.output_keys = tokenizer, keys, output_keys
        self.tokenizer_kwargs = tokenizer_kwargs

    def __call__(self, iterator):
        for rec in iterator:
            for i, k in enumerate(self.keys):
                out = self.output_keys[i] if self.output_keys else k
                rec[out] = self.tokenizer.encode(rec[k], **self.tokenizer_kwargs)
            yield rec


class SequencePacking:
    """Concatenate token lists and cut fixed-length windows (`rewind` tokens of overlap). The
    leftover tokens and the ids of the documents they came from are the operator's state."""

    def __init__(self, length, key="text", rewind=0):
        self.length, self.key, self.rewind = length, key, rewind
        self._tokens, self._dataset_ids, self._sample_ids = [], [], []

    def state_dict(self):
        return {"tokens": list(self._tokens), "packed_dataset_ids": list(self._dataset_ids),
                "packed_sample_ids": list(self._sample_ids)}

    def load_state_dict(self, state):
        self._tokens = list(state["tokens"])
        self._dataset_ids = list(state["packed_dataset_ids"])
        self._sample_ids = list(state["packed_sample_ids"])

    def __call__(self, iterator):
        for rec in iterator:
            self._tokens.extend(rec[self.key])
            meta = rec.get("_meta_", {})
            self._dataset_ids.append(meta.get("dataset_id"))
            self._sample_ids.append(meta.get("sample_id"))
            while len(self._tokens) >= self.length:
                window = self._tokens[: self.length]
                self._tokens = self._tokens[self.length - self.rewind:]
                out = Record({**rec, self.key: window})
                out["_meta_"] = {**meta, "dataset_ids": list(self._dataset_ids),
                                 "sample_ids": list(self._sample_ids)}
                self._dataset_ids = self._dataset_ids[-1:]
                self._sample_ids = self._sample_ids[-1:]
                yield out
            if not self._tokens:
                self._dataset_ids, self._sample_ids = [], []


class AutoregressiveSample:
    """tokens -> input (all but last), target (all but first)."""

    def __init__(self, key="text"):
        self.key = key

    def __call__(self, iterator):
        for rec in iterator:
            rec["input"] = rec[self.key][:-1]
            rec["target"] = rec[self.key][1:]
            yield rec


def collate_list(batch):
    return batch


class Collator:
    """Stack `keys` into tensors (or use a per-key collate function); other fields become lists,
    per-sample `_meta_` goes to `_meta_["samples_meta"]`."""

    def __init__(self, keys=("text",), skip_except_keys=False, collate_fns: dict[str, Callable] | None = None):
        self.keys = keys
        self.skip_except_keys = skip_except_keys
        self.collate_fns = collate_fns or {}

    def __call__(self, batch):
        out = Record()
        out["_meta_"] = {"batch_keys": self.keys}
        for k in self.keys:
            column = [rec[k] for rec in batch]
            out[k] = self.collate_fns[k](column) if k in self.collate_fns else \
                torch.stack([torch.as_tensor(v) for v in column], 0)
        if self.skip_except_keys:
            return out
        out["_meta_"]["samples_meta"] = [rec.get("_meta_") for rec in batch if "_meta_" in rec]
        for rec in batch:
            for k, v in rec.items():
                if k in self.keys or k == "_meta_":
                    continue
                out.setdefault(k, []).append(v)
        return out
