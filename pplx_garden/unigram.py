"""Unigram (SentencePiece-style) tokenizer encoder, CPU, multithreaded.

``Engine`` loads a HuggingFace ``tokenizer.json`` (Precompiled-charsmap normaliser,
Metaspace pre-tokenizer, Unigram model without byte fallback, special added tokens only)
and encodes text to token ids with the native implementation in ``csrc/unigram``. It has
the behaviour of the reference's ``pplx-unigram`` crate (pplx-unigram/src/lib.rs:10-35,
docs/unigram.md); the reference exposes that crate to Rust callers only.
"""

from __future__ import annotations

import os
from typing import Sequence, Union

from pplx_garden._native import UnigramEngine as _UnigramEngine


class Engine:
    def __init__(self, native: _UnigramEngine) -> None:
        self._native = native

    @classmethod
    def from_hf_json_path(cls, path: Union[str, os.PathLike]) -> "Engine":
        return cls(_UnigramEngine.from_hf_json_path(os.fspath(path)))

    @classmethod
    def from_hf_json_bytes(cls, data: Union[bytes, str]) -> "Engine":
        if isinstance(data, str):
            data = data.encode("utf-8")
        return cls(_UnigramEngine.from_hf_json_bytes(data))

    @property
    def vocab_size(self) -> int:
        """Base vocabulary plus added tokens (largest id + 1)."""
        return self._native.vocab_size

    @property
    def unk_id(self) -> int:
        return self._native.unk_id

    def encode(self, text: str) -> list[int]:
        return self._native.encode(text)

    def encode_batch(self, texts: Sequence[str], num_threads: int = 0) -> list[list[int]]:
        """Encode many texts in parallel (``num_threads`` 0 = one per hardware thread).
        The GIL is released while the worker threads run."""
        return self._native.encode_batch(list(texts), num_threads)

    def encode_batch_flat(self, texts: Sequence[str], num_threads: int = 0):
        """Like ``encode_batch`` but returns ``(ids, offsets)`` as numpy arrays (int32 [total tokens],
        int64 [len(texts) + 1]; text i is ``ids[offsets[i]:offsets[i + 1]]``): no Python integer per
        token, which is what bounds ``encode_batch`` on large batches."""
        return self._native.encode_batch_flat(list(texts), num_threads)

    def normalize(self, text: str) -> str:
        return self._native.normalize(text)
