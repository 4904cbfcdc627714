"""The token mask of constrained decoding on the host: the bitset and its limits (the reference's
cases, crates/mrun-engine/src/engine.rs:948-990), and what the scheduler does with a request whose
mask cannot be used."""
from __future__ import annotations

import numpy as np

from mrun_b200.sampling import TokenMask


def test_token_mask_allows_only_set_tokens():
    mask = TokenMask.none_allowed(130)
    assert mask.is_none()
    for token in (0, 129, 500, -1):
        mask.allow(token)
    assert mask.is_allowed(0) and mask.is_allowed(129)
    assert not mask.is_allowed(1) and not mask.is_allowed(500) and not mask.is_allowed(-1)
    assert not mask.is_none() and mask.allowed() == [0, 129] and mask.vocab == 130


def test_token_mask_from_words_reads_a_32_bit_bitset():
    mask = TokenMask.from_words([0b101, 1 << 31, 0xFFFFFFFF], 70)       # bits at or above 70 are ignored
    assert mask.allowed() == [0, 2, 63, 64, 65, 66, 67, 68, 69]
    assert TokenMask.from_words([], 70).is_none()                        # missing words allow nothing
    assert TokenMask.from_words([1, 2, 3, 4, 5], 40).allowed() == [0, 33]    # words past the vocabulary are dropped
    assert TokenMask.of([3, 3, 64], 65).words.tolist() == [8, 0, 1] and TokenMask.of([3], 65).words.dtype == np.uint32
