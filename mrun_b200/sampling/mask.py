"""Allowed next tokens for constrained decoding: a bitset over the vocabulary, bit ``i`` set =
token ``i`` may be sampled (the reference's ``TokenMask``, crates/mrun-engine/src/engine.rs:383-460).
A mask narrower than the model's logits (a tokenizer's vocabulary below the padded embedding)
leaves the rest disallowed; a wider one is refused; one that allows nothing ends the request
(``EmptyMask`` / ``MaskTooWide``, crates/mrun-engine/src/engine.rs:571-576).  The sampler sets the
logits of every other token to -inf before its filters and its draw, which is the reference's
``where(mask, logprobs, -inf)`` (crates/mrun-engine/src/sample.rs:104-116): the filters and the
draw see only differences of log-probabilities among the allowed tokens.
"""
from __future__ import annotations

from typing import Iterable

import numpy as np


class TokenMask:
    def __init__(self, words: np.ndarray, vocab: int):
        self.words, self.vocab = words, int(vocab)

    @classmethod
    def none_allowed(cls, vocab: int) -> "TokenMask":
        if vocab < 0:
            raise ValueError(f"a token mask over {vocab} tokens")
        return cls(np.zeros(-(-int(vocab) // 32), dtype=np.uint32), vocab)

    @classmethod
    def from_words(cls, words: Iterable[int], vocab: int) -> "TokenMask":
        """From a bitset in 32-bit words (bit ``i % 32`` of word ``i // 32`` allows token ``i``),
        the layout grammar engines produce.  Missing words allow nothing; bits at or above
        ``vocab`` are ignored."""
        mask = cls.none_allowed(vocab)
        given = np.asarray(list(words), dtype=np.uint64).astype(np.uint32)[:len(mask.words)]
        mask.words[:len(given)] = given
        if vocab % 32 and len(mask.words):
            mask.words[-1] &= np.uint32((1 << (vocab % 32)) - 1)
        return mask

    @classmethod
    def of(cls, tokens: Iterable[int], vocab: int) -> "TokenMask":
        mask = cls.none_allowed(vocab)
        for token in tokens:
            mask.allow(token)
        return mask

    def allow(self, token: int) -> None:
        token = int(token)
        if 0 <= token < self.vocab:
            self.words[token // 32] |= np.uint32(1 << (token % 32))

    def is_allowed(self, token: int) -> bool:
        token = int(token)
        return 0 <= token < self.vocab and bool(self.words[token // 32] >> np.uint32(token % 32) & np.uint32(1))

    def is_none(self) -> bool:
        """Whether no token is allowed."""
        return not self.words.any()

    def allowed(self) -> list:
        return [int(i) for i in np.flatnonzero(np.unpackbits(self.words.view(np.uint8), bitorder="little")[:self.vocab])]
