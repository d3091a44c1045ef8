"""Supervised fine-tuning samples and pad-aware packing (reference: projects/sft/preprocess.py:6-296).

`SFTSample` tokenises prompt and response separately and masks the prompt out of the target.
`SFTSequencePacking` fills fixed-length rows with whole samples: a sample that does not fit
closes the current row (padded) and opens the next; a sample longer than a row is truncated (or
continued in following rows). Rows can carry per-document `position_ids` and cumulative
`document_offsets` for document-masked attention.
"""

from __future__ import annotations

import torch

from halite_b200.data.record import Record


class SFTSample:
    def __init__(self, prompt_key, response_key, tokenizer=None, input_key="input", target_key="target",
                 prompt_map_fn=None, response_map_fn=None, prompt_tokenizer_kwargs=None,
                 response_tokenizer_kwargs=None, ignore_index=-100):
        self.prompt_key, self.response_key = prompt_key, response_key
        self.tokenizer = tokenizer
        self.input_key, self.target_key = input_key, target_key
        self.prompt_map_fn, self.response_map_fn = prompt_map_fn, response_map_fn
        self.prompt_tokenizer_kwargs = prompt_tokenizer_kwargs or {}
        self.response_tokenizer_kwargs = response_tokenizer_kwargs or {}
        self.ignore_index = ignore_index

    def __call__(self, iterator):
        for record in iterator:
            yield self.process(record)

    def process(self, record):
        prompt, response = record[self.prompt_key], record[self.response_key]
        if self.prompt_map_fn is not None:
            prompt = self.prompt_map_fn(prompt)
        if self.response_map_fn is not None:
            response = self.response_map_fn(response)
        p = self.tokenizer.encode(prompt, **self.prompt_tokenizer_kwargs)
        r = self.tokenizer.encode(response, **self.response_tokenizer_kwargs)
        tokens = torch.as_tensor(list(p) + list(r), dtype=torch.int64)
        # next-token targets; prompt positions and the position after the last token are ignored
        target = torch.full_like(tokens, self.ignore_index)
        if len(r) > 0:
            target[max(len(p) - 1, 0):-1] = tokens[max(len(p), 1):]
        record[self.input_key] = tokens
        record[self.target_key] = target
        return record


def length_to_offsets(lengths) -> torch.Tensor:
    return torch.tensor([0] + list(lengths), dtype=torch.int32).cumsum(0).to(torch.int32)


def collate_offsets(offsets, max_len: int) -> torch.Tensor:
    """Stack per-row offset vectors, padding each by repeating its last value."""
    out = torch.zeros(len(offsets), max_len, dtype=torch.int32)
    for i, off in enumerate(offsets):
        n = min(len(off), max_len)
        out[i, :n] = off[:n]
        out[i, n:] = off[-1]
    return out


class SFTSequencePacking:
    def __init__(self, length=None, input_key="input", target_key="target", input_pad=0, target_pad=-100,
                 use_position_ids=False, use_document_offsets=False, use_rest_of_long_sequence=False):
        self.length = length
        self.input_key, self.target_key = input_key, target_key
        self.input_pad, self.target_pad = input_pad, target_pad
        self.use_position_ids, self.use_document_offsets = use_position_ids, use_document_offsets
        self.use_rest_of_long_sequence = use_rest_of_long_sequence
        self._pending = []          # [(input, target, dataset_id, sample_id)] not yet emitted

    # ------------------------------------------------------------------ resumable state
    def state_dict(self):
        return {"input_ids": [p[0] for p in self._pending], "target_ids": [p[1] for p in self._pending],
                "dataset_ids": [p[2] for p in self._pending], "sample_ids": [p[3] for p in self._pending]}

    def load_state_dict(self, state):
        self._pending = list(zip(state["input_ids"], state["target_ids"], state["dataset_ids"], state["sample_ids"]))

    # ------------------------------------------------------------------ packing
    def _emit(self, record, parts, pad):
        inputs = [p[0] for p in parts]
        targets = [p[1] for p in parts]
        if pad > 0:
            inputs.append(torch.full((pad,), self.input_pad, dtype=torch.int64))
            targets.append(torch.full((pad,), self.target_pad, dtype=torch.int64))
        out = {**record, self.input_key: torch.cat(inputs), self.target_key: torch.cat(targets),
               "_tokenized_keys_": (self.input_key, self.target_key)}
        if self.use_document_offsets:
            out["document_offsets"] = length_to_offsets([len(t) for t in inputs])
        if self.use_position_ids:
            out["position_ids"] = torch.cat([torch.arange(len(t)) for t in inputs])
        meta = dict(out.get("_meta_", {}))
        meta.update(dataset_ids=[p[2] for p in parts], sample_ids=[p[3] for p in parts])
        out["_meta_"] = meta
        return Record(out)

    def _take_row(self):
        """Pop the samples of one full row, or None while the pending samples do not yet force
        a row to close."""
        used, parts = 0, []
        for i, (inp, tgt, did, sid) in enumerate(self._pending):
            n = len(inp)
            if used + n <= self.length:
                parts.append((inp, tgt, did, sid))
                used += n
                if used == self.length:
                    self._pending = self._pending[i + 1:]
                    return parts, 0
                continue
            if used > 0:                       # does not fit: close the row with padding
                self._pending = self._pending[i:]
                return parts, self.length - used
            # a single sample longer than a row
            parts.append((inp[:self.length], tgt[:self.length], did, sid))
            rest = self._pending[i + 1:]
            if self.use_rest_of_long_sequence:
                rest = [(inp[self.length:], tgt[self.length:], did, sid)] + rest
            self._pending = rest
            return parts, 0
        return None

    def __call__(self, iterator):
        record = None
        for record in iterator:
            meta = record.get("_meta_", {})
            self._pending.append((record[self.input_key], record[self.target_key], meta.get("dataset_id"),
                                  meta.get("sample_id")))
            while True:
                row = self._take_row()
                if row is None:
                    break
                yield self._emit(record, *row)
        if self._pending and record is not None:
            parts, self._pending = self._pending, []
            used = sum(len(p[0]) for p in parts)
            yield self._emit(record, parts, self.length - used)
