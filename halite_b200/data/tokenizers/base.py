"""Common tokenizer surface (reference: data/tokenizers/*.py): `encode(text, bos=, eos=)`,
`decode(ids)`, `bos_id` / `eos_id` / `pad_id`, `additional_stop_token_ids`, batch helpers."""

from __future__ import annotations


class Tokenizer:
    bos_id: int | None = None
    eos_id: int | None = None
    pad_id: int | None = None
    additional_stop_token_ids: tuple = ()

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def encode(self, text, bos=False, eos=False, **kwargs):
        raise NotImplementedError

    def decode(self, ids, **kwargs):
        raise NotImplementedError

    def encode_batch(self, texts, **kwargs):
        return [self.encode(t, **kwargs) for t in texts]

    def decode_batch(self, batch, **kwargs):
        return [self.decode(ids, **kwargs) for ids in batch]

    @property
    def eos_token_id(self):
        return self.eos_id


class ByteTokenizer(Tokenizer):
    """UTF-8 bytes + (bos, eos, pad): needs no vocabulary file; used by tests and H-Net style
    byte-level models."""

    def __init__(self):
        self.bos_id, self.eos_id, self.pad_id = 256, 257, 258

    @property
    def vocab_size(self):
        return 259

    def encode(self, text, bos=False, eos=False, add_special_tokens=None, **kwargs):
        ids = list(text.encode("utf-8"))
        return ([self.bos_id] if bos else []) + ids + ([self.eos_id] if eos else [])

    def decode(self, ids, **kwargs):
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")
