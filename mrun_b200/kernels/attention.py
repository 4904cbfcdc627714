"""Chooses the attention kernel for a step and launches it.

Every kernel reads keys and values from the pages; the tokens of the step were written there by
the fused norm/rotary/cache kernel just before.  float32 always runs the CUDA-core kernel in
32-bit arithmetic.
"""
from __future__ import annotations

import torch

from . import ops


def paged_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, cache, group, ctx,
                    heads: int, scale: float, window: int) -> torch.Tensor:
    """``q``: the step's queries (row t at ``q_stride * t``, heads contiguous); ``cache``: the
    schedule entry's pages; ``group``: the step's block tables for the cache's group."""
    return ops.paged_attention_generic(q, q_stride, out, cache.k, cache.v, group.block_tables,
                                       ctx.token_slot, ctx.positions, heads, scale, window)
