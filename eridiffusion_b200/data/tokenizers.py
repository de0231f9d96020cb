"""Prompt tokenisers for the text encoders.

Reference: ``HfTokenizer`` over a ``tokenizer.json`` (crates/common/text/src/lib.rs), the CLIP / T5
tokeniser loaders of src/trainers/real_tokenizers.rs (pad / truncate to 77 or 512, BOS / EOS
handling, attention mask from lengths) and the fall-back used by smoke runs when no tokeniser files
are given.

``HfTokenizer`` reads either a single ``tokenizer.json`` (through the ``tokenizers`` library) or a
tokeniser directory (through ``transformers``); both produce ``(ids [B, T] int64, mask [B, T]
bool)`` padded to ``max_length``. ``HashTokenizer`` needs no files: a word-level, deterministic
mapping into the vocabulary, so synthetic pipelines and tests exercise the same code path with
stable ids.
"""
from __future__ import annotations

import hashlib
import os
import re

import torch


class TokenizerError(RuntimeError):
    pass


def pad_or_truncate(ids: list[int], max_length: int, pad_id: int, eos_id: int | None = None):
    """Cut to ``max_length`` (keeping a final EOS when one is defined) and pad on the right.
    Returns (ids, number of real tokens)."""
    if len(ids) > max_length:
        ids = ids[:max_length]
        if eos_id is not None:
            ids[-1] = eos_id
    n = len(ids)
    return ids + [pad_id] * (max_length - n), n


class HfTokenizer:
    def __init__(self, path: str, max_length: int = 77, pad_id: int | None = None):
        self.max_length = max_length
        self._tk = self._hf = None
        if os.path.isdir(path) and not os.path.exists(os.path.join(path, "tokenizer.json")):
            self._load_dir(path)
        else:
            f = os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path
            if not os.path.exists(f):
                raise TokenizerError(f"tokenizer file {f!r} not found")
            from tokenizers import Tokenizer
            self._tk = Tokenizer.from_file(f)
        self.pad_id = pad_id if pad_id is not None else self._default_pad()

    def _load_dir(self, path):
        try:
            from transformers import AutoTokenizer
            self._hf = AutoTokenizer.from_pretrained(path)
        except Exception as e:
            raise TokenizerError(f"cannot load a tokenizer from {path!r}: {e}") from e

    def _default_pad(self):
        if self._hf is not None:
            return self._hf.pad_token_id if self._hf.pad_token_id is not None else (self._hf.eos_token_id or 0)
        for tok in ("<pad>", "<|endoftext|>", "[PAD]", "</s>"):
            i = self._tk.token_to_id(tok)
            if i is not None:
                return i
        return 0

    @property
    def vocab_size(self):
        return len(self._hf) if self._hf is not None else self._tk.get_vocab_size()

    def encode(self, texts, max_length: int | None = None):
        if isinstance(texts, str):
            texts = [texts]
        T = max_length or self.max_length
        rows, lens = [], []
        for t in texts:
            ids = (self._hf(t, add_special_tokens=True)["input_ids"] if self._hf is not None
                   else self._tk.encode(t, add_special_tokens=True).ids)
            eos = self._hf.eos_token_id if self._hf is not None else None
            ids, n = pad_or_truncate(list(ids), T, self.pad_id, eos)
            rows.append(ids)
            lens.append(n)
        ids = torch.tensor(rows, dtype=torch.long)
        mask = torch.arange(T)[None, :] < torch.tensor(lens)[:, None]
        return ids, mask

    __call__ = encode

    def decode(self, ids):
        ids = [int(i) for i in ids if int(i) != self.pad_id]
        return self._hf.decode(ids, skip_special_tokens=True) if self._hf is not None else self._tk.decode(ids)


class HashTokenizer:
    """File-free stand-in: lower-cased words and punctuation marks hash (SHA-256) into
    ``[first_id, vocab_size)``; BOS / EOS are added when given. Same text -> same ids on every
    machine and run."""

    _split = re.compile(r"[\w']+|[^\w\s]")

    def __init__(self, vocab_size: int = 49408, max_length: int = 77, bos_id: int | None = None,
                 eos_id: int | None = None, pad_id: int = 0, first_id: int = 1000):
        if first_id >= vocab_size:
            first_id = min(3, vocab_size - 1)
        self.vocab_size, self.max_length = vocab_size, max_length
        self.bos_id, self.eos_id, self.pad_id, self.first_id = bos_id, eos_id, pad_id, first_id

    @classmethod
    def clip(cls, max_length=77):
        return cls(49408, max_length, bos_id=49406, eos_id=49407, pad_id=49407)

    @classmethod
    def t5(cls, max_length=512):
        return cls(32128, max_length, bos_id=None, eos_id=1, pad_id=0)

    def word_id(self, word: str) -> int:
        h = int.from_bytes(hashlib.sha256(word.encode()).digest()[:8], "little")
        return self.first_id + h % (self.vocab_size - self.first_id)

    def encode(self, texts, max_length: int | None = None):
        if isinstance(texts, str):
            texts = [texts]
        T = max_length or self.max_length
        rows, lens = [], []
        for t in texts:
            ids = [self.word_id(w) for w in self._split.findall(t.lower())]
            if self.bos_id is not None:
                ids = [self.bos_id] + ids
            if self.eos_id is not None:
                ids = ids + [self.eos_id]
            ids, n = pad_or_truncate(ids, T, self.pad_id, self.eos_id)
            rows.append(ids)
            lens.append(n)
        return torch.tensor(rows, dtype=torch.long), torch.arange(T)[None, :] < torch.tensor(lens)[:, None]

    __call__ = encode


def load_tokenizer(path: str | None, kind: str = "clip", max_length: int | None = None):
    """``path`` None or empty: the hash tokeniser for ``kind`` (``clip`` | ``t5``); else files."""
    default_len = {"clip": 77, "t5": 512}.get(kind, 77)
    if not path:
        return HashTokenizer.t5(max_length or default_len) if kind == "t5" else HashTokenizer.clip(max_length or default_len)
    return HfTokenizer(path, max_length or default_len)
