"""SentencePiece tokenizer (reference: data/tokenizers/sentencepiece.py)."""

from __future__ import annotations

from halite_b200.data.tokenizers.base import Tokenizer


class SentencePieceTokenizer(Tokenizer):
    def __init__(self, model_path):
        import sentencepiece as spm

        self.model_path = model_path
        self.sp = spm.SentencePieceProcessor(model_file=model_path)
        self.bos_id, self.eos_id, self.pad_id = self.sp.bos_id(), self.sp.eos_id(), self.sp.pad_id()

    @property
    def vocab_size(self):
        return self.sp.vocab_size()

    def encode(self, text, bos=False, eos=False, add_special_tokens=None, **kwargs):
        ids = self.sp.encode(text)
        return ([self.bos_id] if bos else []) + ids + ([self.eos_id] if eos else [])

    def decode(self, ids, **kwargs):
        return self.sp.decode(list(ids))
