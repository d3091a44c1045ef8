"""Llama-3 tiktoken tokenizer (reference: data/tokenizers/llama3.py:1-214): BPE ranks from the
model file, 256 reserved special tokens, the Llama-3 split pattern; long inputs are encoded in
chunks to bound the regex cost."""

from __future__ import annotations

import os

from halite_b200.data.tokenizers.base import Tokenizer

_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
            r"\s*[\r\n]+|\s+(?!\S)|\s+")
_N_RESERVED = 256
_MAX_CHARS = 400_000


class Llama3Tokenizer(Tokenizer):
    def __init__(self, model_path=None):
        self.model_path = model_path
        self._model = None
        if model_path is not None and os.path.exists(model_path):
            self._load()

    def _load(self):
        import tiktoken
        from tiktoken.load import load_tiktoken_bpe

        ranks = load_tiktoken_bpe(self.model_path)
        n = len(ranks)
        named = ["<|begin_of_text|>", "<|end_of_text|>", "<|reserved_special_token_0|>",
                 "<|reserved_special_token_1|>", "<|finetune_right_pad_id|>", "<|step_id|>",
                 "<|start_header_id|>", "<|end_header_id|>", "<|eom_id|>", "<|eot_id|>", "<|python_tag|>"]
        named += [f"<|reserved_special_token_{2 + i}|>" for i in range(_N_RESERVED - len(named))]
        self.special = {tok: n + i for i, tok in enumerate(named)}
        self._model = tiktoken.Encoding(name=os.path.basename(self.model_path), pat_str=_PATTERN,
                                        mergeable_ranks=ranks, special_tokens=self.special)
        self.bos_id = self.special["<|begin_of_text|>"]
        self.eos_id = self.special["<|end_of_text|>"]
        self.pad_id = self.special["<|finetune_right_pad_id|>"]
        self.additional_stop_token_ids = (self.special["<|eom_id|>"], self.special["<|eot_id|>"])

    @property
    def model(self):
        if self._model is None:
            self._load()
        return self._model

    @property
    def vocab_size(self):
        return self.model.n_vocab

    def encode(self, text, bos=False, eos=False, allowed_special=(), disallowed_special=(), **kwargs):
        ids = []
        for start in range(0, len(text), _MAX_CHARS):
            ids.extend(self.model.encode(text[start:start + _MAX_CHARS], allowed_special=set(allowed_special) or set(),
                                         disallowed_special=disallowed_special))
        return ([self.bos_id] if bos else []) + ids + ([self.eos_id] if eos else [])

    def decode(self, ids, **kwargs):
        return self.model.decode(list(ids))
