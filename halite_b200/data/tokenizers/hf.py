"""Hugging Face `tokenizers` / `transformers` backed tokenizer (reference:
data/tokenizers/hf.py)."""

from __future__ import annotations

from halite_b200.data.tokenizers.base import Tokenizer


class HFTokenizer(Tokenizer):
    def __init__(self, model_path, bos_token=None, eos_token=None, additional_stop_tokens=(), **kwargs):
        from transformers import AutoTokenizer

        self.model_path = model_path
        self.tok = AutoTokenizer.from_pretrained(model_path, **kwargs)
        self.bos_id = self.tok.convert_tokens_to_ids(bos_token) if bos_token else self.tok.bos_token_id
        self.eos_id = self.tok.convert_tokens_to_ids(eos_token) if eos_token else self.tok.eos_token_id
        self.pad_id = self.tok.pad_token_id
        self.additional_stop_token_ids = tuple(self.tok.convert_tokens_to_ids(t) for t in additional_stop_tokens)

    @property
    def vocab_size(self):
        return len(self.tok)

    def encode(self, text, bos=False, eos=False, add_special_tokens=False, **kwargs):
        ids = self.tok.encode(text, add_special_tokens=add_special_tokens, **kwargs)
        if bos and self.bos_id is not None and (not ids or ids[0] != self.bos_id):
            ids = [self.bos_id] + ids
        if eos and self.eos_id is not None:
            ids = ids + [self.eos_id]
        return ids

    def encode_batch(self, texts, bos=False, eos=False, **kwargs):
        out = self.tok(list(texts), add_special_tokens=False, **kwargs)["input_ids"]
        return [([self.bos_id] if bos and self.bos_id is not None else []) + ids +
                ([self.eos_id] if eos and self.eos_id is not None else []) for ids in out]

    def decode(self, ids, skip_special_tokens=True, **kwargs):
        return self.tok.decode(ids, skip_special_tokens=skip_special_tokens, **kwargs)

    def decode_batch(self, batch, skip_special_tokens=True, **kwargs):
        return self.tok.batch_decode(batch, skip_special_tokens=skip_special_tokens, **kwargs)
