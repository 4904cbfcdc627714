"""Chooses the attention kernel for a step and launches it.

Every kernel reads keys and values from the pages; the tokens of the step were written there by
the fused norm/rotary/cache kernel just before.

* float32, or a shape the tensor-core kernels refuse: the CUDA-core kernel in 32-bit arithmetic.
* bfloat16, every segment a single token: the split-key decode kernel (scratch for the partial
  results of the splits, merged by a second kernel).
* bfloat16 otherwise: the tiled prefill kernel over (tokens x group heads) row tiles.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import lib as _lib
from . import ops
from .ops import _c_float, _c_int, _c_long, _ptr, _stream

MAX_SPLITS = 64
COUNTER_CAPACITY = 1 << 16     # (token, kv head) pairs of one decode launch that may be split

_counters = {}                 # device -> int32 zeros, handed to every split launch
_slots = {}                    # head size -> blocks of the decode kernel resident on the device


def _decode_slots(head_dim: int, library) -> int:
    slots = _slots.get(head_dim)
    if slots is None:
        query = library._dll.mrun_attn_decode_occupancy
        query.restype = ctypes.c_int
        per_sm = max(1, query())
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        slots = _slots[head_dim] = per_sm * sms
    return slots


def _split_counters(device: torch.device) -> torch.Tensor:
    """Zeroed counters the decode kernel's splits meet at; the kernel leaves them zero.  One
    buffer per device, never reallocated, so captured graphs may keep its address."""
    counters = _counters.get(device)
    if counters is None:
        counters = _counters[device] = torch.zeros(COUNTER_CAPACITY, dtype=torch.int32, device=device)
    return counters


def supports_tensor_cores(dtype: torch.dtype, head_dim: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and group <= 64


def decode_splits(tokens: int, kv_heads: int, max_kv_len: int, slots: int):
    """(splits, min_tiles): how many ways the keys of a token may be split and the fewest 64-key
    tiles a split takes.  Few (token, kv head) pairs: as many splits as fill the device once, four
    tiles each at least.  More pairs than the device holds at a time: up to four rounds of blocks,
    so that the last, partly filled round costs little, but only for contexts long enough to give
    every split sixteen tiles.  (Measured on B200 at head size 128.)  The kernel applies
    ``min_tiles`` to each token's own context, so short contexts use fewer splits."""
    pairs = max(1, tokens * kv_heads)
    blocks = max(1, -(-max_kv_len // 64))
    if pairs > COUNTER_CAPACITY:
        return 1, 1
    if pairs < slots:
        want, min_tiles = slots // pairs, 4
    else:
        want, min_tiles = -(-4 * slots // pairs), 16
    return max(1, min(want, -(-blocks // min_tiles), MAX_SPLITS)), min_tiles


def prefill_tiles(ctx, tokens_per_tile: int):
    """(first token row, token count) of every row tile, as device int32 arrays; made once per
    step and group size."""
    key = ("attention_tiles", tokens_per_tile)
    tiles = ctx.shared.get(key)
    if tiles is None:
        first, count = [], []
        for seg in ctx.segments:
            for t0 in range(0, seg.q_len, tokens_per_tile):
                first.append(seg.q_start + t0)
                count.append(min(tokens_per_tile, seg.q_len - t0))
        n = len(first)
        both = ctx.upload(np.asarray(first + count, dtype=np.int32))
        tiles = ctx.shared[key] = (both[:n], both[n:], n)
    return tiles


def decode_fuses_input(ctx, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether this step's attention takes q, k and v raw and norms, rotates and stores them itself
    (every segment a single token, bfloat16, a group that the split-key kernel takes)."""
    ratio = heads // kv_heads
    return ctx.all_decode and ratio <= 16 and supports_tensor_cores(dtype, head_dim, ratio)


def paged_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, cache, group, ctx,
                    heads: int, scale: float, window: int, raw=None) -> torch.Tensor:
    """``q``: the step's queries (row t at ``q_stride * t``, heads contiguous); ``cache``: the
    schedule entry's pages; ``group``: the step's view of the cache's group.  ``raw``, only where
    :func:`decode_fuses_input` holds: ``(q_weight, k_weight, eps, rot, rotary_dim, slots)`` for a
    ``q`` that is the projection's raw [q | k | v] rows."""
    pages, kv_heads, page_size, head_dim = cache.k.shape
    ratio = heads // kv_heads
    if not supports_tensor_cores(q.dtype, head_dim, ratio):
        return ops.paged_attention_generic(q, q_stride, out, cache.k, cache.v, group.block_tables,
                                           ctx.token_slot, ctx.positions, heads, scale, window)
    library = _lib.attention(head_dim)
    tokens = ctx.num_tokens
    common = (_ptr(cache.k), _ptr(cache.v), _ptr(group.block_tables), _c_int(group.max_blocks),
              _ptr(ctx.token_slot), _ptr(ctx.positions))
    tail = (_c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page_size), _c_float(scale),
            _c_int(window), _stream())
    if ctx.all_decode and ratio <= 16:
        splits, min_tiles = decode_splits(tokens, kv_heads, ctx.max_kv_len, _decode_slots(head_dim, library))
        part_o = part_ml = counters = None
        if splits > 1:
            part_o = torch.empty((tokens, heads, splits, head_dim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((tokens, heads, splits, 2), dtype=torch.float32, device=q.device)
            counters = _split_counters(q.device)
        fused = (_c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None))
        if raw is not None:
            q_weight, k_weight, eps, rot, rotary_dim, slots = raw
            fused = (_c_int(1), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(rot), _c_int(rotary_dim),
                     _ptr(slots))
        library.call("mrun_attn_decode", _ptr(q), _c_long(q_stride), _ptr(out), *common, _c_int(tokens),
                     _ptr(part_o), _ptr(part_ml), _ptr(counters), _c_int(splits), _c_int(min_tiles), *tail[:-1],
                     *fused, tail[-1])
        return out
    if raw is not None:
        raise ValueError("raw q, k, v rows are taken by the decode kernel only")
    first, count, n_tiles = prefill_tiles(ctx, 64 // ratio)
    if tokens > ctx.real_tokens:
        out[ctx.real_tokens:].zero_()
    library.call("mrun_attn_prefill", _ptr(q), _c_long(q_stride), _ptr(out), *common, _ptr(first),
                 _ptr(count), _c_int(n_tiles), *tail)
    return out
