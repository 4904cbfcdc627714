"""The tiny configurations the tests run on.  They differ in every size and option: head counts and
groups, sizes that are no power of two, number of layers, vocabulary, the norms' eps, rope base,
tied or untied head, norm weights, page size.  A and B have small heads (the mma.sync attention
kernels), C has heads of 64 and E heads of 128 (the TMA and tcgen05 attention kernels), D sizes
that are no multiple of 8.

The weights' standard deviations (0.06 to 0.08) are larger than the 0.02 of the measured shapes: at
widths of 64 to 256 that keeps the logits a few units wide, so that an error in a single head or
layer shows against the tolerance, which is relative to the largest logit of the configuration."""
from __future__ import annotations

import numpy as np

TINY = {
    "A": dict(
        config=dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=16, intermediate_size=128, vocab_size=256, max_position_embeddings=1024,
                    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True),
        seed=11, std=0.08, norm_noise=0.0, page_size=16),
    "B": dict(
        config=dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=3,
                    head_dim=32, intermediate_size=200, vocab_size=509, max_position_embeddings=2048,
                    rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False),
        seed=23, std=0.06, norm_noise=0.1, page_size=8),
    # heads of 64: the sizes the TMA decode attention and the tcgen05 prefill attention take
    "C": dict(
        config=dict(num_hidden_layers=2, hidden_size=160, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=64, intermediate_size=224, vocab_size=300, max_position_embeddings=4096,
                    rms_norm_eps=3e-6, rope_theta=500000.0, tie_word_embeddings=False),
        seed=37, std=0.07, norm_noise=0.05, page_size=16),
    # sizes that fit no vector width: a width and an intermediate size that are no multiple of 8, one
    # kv head for eight query heads, heads of 48, an odd vocabulary, pages of four tokens
    "D": dict(
        config=dict(num_hidden_layers=2, hidden_size=100, num_attention_heads=8, num_key_value_heads=1,
                    head_dim=48, intermediate_size=150, vocab_size=301, max_position_embeddings=1024,
                    rms_norm_eps=2e-5, rope_theta=50000.0, tie_word_embeddings=True),
        seed=41, std=0.08, norm_noise=0.1, page_size=4),
    # heads of 128, twice the width in heads (heads x head size != width): the head size of the
    # measured shapes, with its three-stage TMA ring and the tcgen05 tiles of 128
    "E": dict(
        config=dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=128, intermediate_size=384, vocab_size=411, max_position_embeddings=2048,
                    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False),
        seed=53, std=0.06, norm_noise=0.1, page_size=16),
}


def tiny_config(name: str):
    from mrun_b200.config import Qwen3Config
    return Qwen3Config(**TINY[name]["config"])


def make_folder(name: str, folder: str, dtype: str = "bfloat16") -> str:
    from mrun_b200.weights import write_random_model
    t = TINY[name]
    return write_random_model(tiny_config(name), folder, seed=t["seed"], std=t["std"],
                              norm_noise=t["norm_noise"], dtype=dtype)


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()


# Error bounds, relative to the largest magnitude of the plain implementation's logits.
# float32: products of a few hundred terms over a handful of layers; bfloat16: 8 bits of mantissa
# in activations, weights and the cache.
TOLERANCE = {"float32": 2e-5, "bfloat16": 4e-2}


def rel_error(got: np.ndarray, want: np.ndarray) -> float:
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / np.max(np.abs(want)))
