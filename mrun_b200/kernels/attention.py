"""Chooses the attention kernel for a step and launches it.

Every kernel reads keys and values from the pages; the tokens of the step were written there by
the fused norm/rotary/cache kernel just before.

* float32, or a shape the tensor-core kernels refuse: the CUDA-core kernel in 32-bit arithmetic.
* bfloat16, every segment a single token: a decode kernel.  Head sizes 64 and 128 with
  power-of-two pages, few pairs and contexts that are not long: a thread-block cluster a
  (token, kv head) pair, which cuts the pair's tiles among its blocks and merges through
  distributed shared memory (no plan, no scratch).  Otherwise the planned kernel, which deals the
  key tiles of all pairs to as many blocks as the device holds (scratch for the partial results
  of pairs shared between blocks, merged by the block that finishes last): tiles brought by TMA
  into a ring for those head and page sizes, else copied with cp.async.
* bfloat16 otherwise: a step with prompt portions.  Its single-token segments (the decoding
  requests beside the prompts) go through the TMA decode kernel as a selection of the step's rows
  where that kernel takes the shape; the rest as follows.  Head sizes 64 and 128: the tcgen05 kernel (128-row tiles
  of tokens x group heads, accumulators in tensor memory) for every segment with more rows than
  one tile of the older kernel; the mma.sync kernel (64-row tiles) for the rest of the step (the
  single decode tokens of a mixed step, short tails) and for the other head sizes.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import lib as _lib
from . import ops
from .ops import _c_float, _c_int, _c_long, _ptr, _stream

COUNTER_CAPACITY = 1 << 16     # (token, kv head) pairs of one decode launch that may be split

_counters = {}                 # device -> int32 zeros, handed to every split launch
_slots = {}                    # head size -> blocks of the decode kernel resident on the device


def _decode_slots(head_dim: int, library, tma_group: int = 0) -> int:
    """Blocks of the decode kernel that the device holds at once: the cp.async kernel's, or, with
    ``tma_group`` query heads per kv head, the TMA kernel's."""
    slots = _slots.get((head_dim, tma_group))
    if slots is None:
        if tma_group:
            per_sm = max(1, int(library._dll.mrun_attn_decode_tma_occupancy(_c_int(tma_group))))
        else:
            query = library._dll.mrun_attn_decode_occupancy
            query.restype = ctypes.c_int
            per_sm = max(1, query())
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        slots = _slots[(head_dim, tma_group)] = per_sm * sms
    return slots


TMA_DECODE = True        # False: the cp.async kernel for every decode step (tests compare the two)
_tma_decode = {}


def decode_uses_tma(library, head_dim: int, ratio: int, page_size: int) -> bool:
    """Head sizes 64 and 128, pages of a power-of-two size (the kernel copies whole pages by TMA)."""
    if not TMA_DECODE or ratio > 16 or page_size & (page_size - 1):
        return False
    have = _tma_decode.get(head_dim)
    if have is None:
        have = _tma_decode[head_dim] = bool(library._dll.mrun_attn_decode_tma_available())
    return have


def decode_slots(head_dim: int, ratio: int, page_size: int) -> int:
    library = _lib.attention(head_dim)
    return _decode_slots(head_dim, library, ratio if decode_uses_tma(library, head_dim, ratio, page_size) else 0)


def _split_counters(device: torch.device) -> torch.Tensor:
    """Zeroed counters the decode kernel's splits meet at; the kernel leaves them zero.  One
    buffer per device, never reallocated, so captured graphs may keep its address."""
    counters = _counters.get(device)
    if counters is None:
        counters = _counters[device] = torch.zeros(COUNTER_CAPACITY, dtype=torch.int32, device=device)
    return counters


CLUSTER_DECODE = True    # False: the planned kernel for every decode step (tests compare the two)
MAX_CLUSTER = 16


def decode_cluster(library, head_dim: int, ratio: int, page_size: int, tokens: int, kv_heads: int,
                   max_kv_len: int) -> int:
    """Blocks of a thread-block cluster that takes one (token, kv head) pair of a decode step, or
    0 where the planned kernel runs instead.  The cluster kernel takes steps whose pairs fill at
    most half the device (each pair is then cut into as many pieces as fit), groups of up to 8,
    and contexts short enough for its pieces: a cluster has at most 16 blocks, so beyond 32 tiles
    a block (8 where the clusters leave a fifth of the device or more empty) the planned kernel,
    which cuts a pair into up to 32 pieces, spreads a long context further."""
    if not CLUSTER_DECODE or ratio > 8 or not decode_uses_tma(library, head_dim, ratio, page_size):
        return 0
    pairs = tokens * kv_heads
    slots = _decode_slots(head_dim, library, ratio)
    if pairs < 1 or 2 * pairs > slots:
        return 0
    cluster = 1
    while cluster < 8 and 2 * cluster * pairs <= slots:
        cluster *= 2
    # sixteen blocks share a part of the device that holds two such clusters: only where the
    # clusters of the step fill at most half of it
    if cluster == 8 and MAX_CLUSTER >= 16 and 32 * pairs <= slots:
        cluster = 16
    tiles_a_block = -(-(-(-max(1, max_kv_len) // 64)) // cluster)
    if tiles_a_block > (32 if 5 * cluster * pairs >= 4 * slots else 8):
        return 0
    return cluster


def supports_tensor_cores(dtype: torch.dtype, head_dim: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and group <= 64


MIN_TILES = 2      # the fewest 64-key tiles a block of the decode kernel takes


MAX_SPLITS = 32    # the most blocks one (token, kv head) pair is cut into when a step has few pairs


def decode_launch(tokens: int, kv_heads: int, slots: int):
    """(blocks, splits) of a decode step of the planned kernel.  More (token, kv head) pairs than
    the device holds blocks: all its blocks, the tiles dealt evenly across pairs (splits = 0).
    Else every block stays with one pair, since a block that never changes pair has no partial
    result to hand over: the launch fills the device once, every kv head has the same number of
    blocks, and the plan deals them to the head's pairs by their length, at most ``splits`` to
    one pair."""
    pairs = tokens * kv_heads
    if pairs > slots:
        # k pairs a block where that leaves at least four fifths of the blocks busy: with equal
        # contexts every block then takes whole pairs and hands nothing over
        k = -(-pairs // slots)
        aligned = -(-pairs // k)
        return (aligned if 5 * aligned >= 4 * slots else slots), 0
    per_head = max(tokens, min(slots // kv_heads, tokens * MAX_SPLITS))
    return per_head * kv_heads, MAX_SPLITS


def decode_plan(ctx, library, window: int, kv_heads: int, blocks: int, splits: int, positions=None):
    """The step's plan for the decode kernel: tiles per token as a prefix sum (int32, tokens + 1;
    with ``splits`` also the blocks per token as a prefix sum and the tiles a block takes) and
    what each of ``blocks`` blocks starts with (int32, 8 per block).  Made once per step for
    a window, a number of kv heads and a launch shape.  ``positions``: those of a selection of the
    step's tokens instead of all of them."""
    key = ("decode_plan", window, kv_heads, blocks, splits, positions is not None)
    plan = ctx.shared.get(key)
    if plan is None:
        if positions is None:
            positions = ctx.positions
        n = positions.shape[0]
        prefix = torch.empty(2 * (n + 1) + 1, dtype=torch.int32, device=positions.device)
        assignment = torch.empty(blocks * 8, dtype=torch.int32, device=positions.device)
        library.call("mrun_attn_decode_plan", _ptr(positions), _c_int(n), _c_int(window),
                     _c_int(kv_heads), _c_int(blocks), _c_int(MIN_TILES), _c_int(splits), _ptr(prefix),
                     _ptr(assignment), _stream())
        plan = ctx.shared[key] = (prefix, assignment)
    return plan


def prefill_tiles(ctx, tokens_per_tile: int, longer_than: int = 0, up_to: int = 1 << 30):
    """(first token row, token count) of every row tile of the segments with more than
    ``longer_than`` and at most ``up_to`` tokens, the tiles with the longest contexts first, as
    device int32 arrays; made once per step and choice of sizes."""
    key = ("attention_tiles", tokens_per_tile, longer_than, up_to)
    tiles = ctx.shared.get(key)
    if tiles is None:
        found = []
        for seg in ctx.segments:
            if not longer_than < seg.q_len <= up_to:
                continue
            for t0 in range(0, seg.q_len, tokens_per_tile):
                count = min(tokens_per_tile, seg.q_len - t0)
                found.append((seg.pos_start + t0 + count, seg.q_start + t0, count))
        # The tile with the most keys before it first: the kernels start their blocks in this
        # order, so the long tiles are under way while the short ones fill the gaps (a stable
        # sort: the order depends on the step's segments only).
        found.sort(key=lambda tile: -tile[0])
        first, count = [tile[1] for tile in found], [tile[2] for tile in found]
        n = len(first)
        both = ctx.upload(np.asarray(first + count, dtype=np.int32))
        tiles = ctx.shared[key] = (both[:n], both[n:], n)
    return tiles


def single_tokens(ctx):
    """The single-token segments of a step that also carries prompt portions, as device int32
    arrays (rows, positions, state slots) and their number; made once per step."""
    found = ctx.shared.get("single_tokens")
    if found is None:
        singles = [seg for seg in ctx.segments if seg.q_len == 1]
        n = len(singles)
        if n:
            packed = ctx.upload(np.asarray([seg.q_start for seg in singles] + [seg.pos_start for seg in singles]
                                           + [seg.slot for seg in singles], dtype=np.int32))
            found = (packed[:n], packed[n:2 * n], packed[2 * n:], n)
        else:
            found = (None, None, None, 0)
        ctx.shared["single_tokens"] = found
    return found


def decode_fuses_input(ctx, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, page_size: int = 16) -> bool:
    """Whether this step's attention takes q, k and v raw and norms, rotates and stores them itself:
    every segment a single token, bfloat16 and a group that the split-key kernel takes.  A block
    that walks from pair to pair redoes the input work at every change, which costs less than the
    stand-alone kernel's launch."""
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
        if tokens * kv_heads > COUNTER_CAPACITY:
            raise ValueError(f"a decode step of {tokens} tokens x {kv_heads} kv heads exceeds {COUNTER_CAPACITY} pairs")
        fused = (_c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None))
        if raw is not None:
            q_weight, k_weight, eps, rot, rotary_dim, slots = raw
            fused = (_c_int(1), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(rot), _c_int(rotary_dim),
                     _ptr(slots))
        cluster = decode_cluster(library, head_dim, ratio, page_size, tokens, kv_heads, ctx.max_kv_len)
        if cluster:
            status = ops.status_word(q.device, "attn_decode_tma", {1: "the TMA producer", 2: "the consumer warps"})
            library.call("mrun_attn_decode_cluster", _ptr(q), _c_long(q_stride), _ptr(out), *common, _c_int(tokens),
                         _c_int(cluster), *tail[:-1], *fused, _ptr(None), _c_long(pages), _ptr(status), tail[-1])
            return out
        tma = decode_uses_tma(library, head_dim, ratio, page_size)
        blocks, splits = decode_launch(tokens, kv_heads, decode_slots(head_dim, ratio, page_size))
        part_o = torch.empty((blocks, 2, 16, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((blocks, 2, 16, 2), dtype=torch.float32, device=q.device)
        prefix, assignment = decode_plan(ctx, library, window, kv_heads, blocks, splits)
        extra = ()
        if tma:
            status = ops.status_word(q.device, "attn_decode_tma", {1: "the TMA producer", 2: "the consumer warps"})
            extra = (_ptr(None), _c_long(pages), _ptr(status))
        library.call("mrun_attn_decode_tma" if tma else "mrun_attn_decode", _ptr(q), _c_long(q_stride), _ptr(out),
                     *common, _ptr(prefix), _ptr(assignment), _c_int(tokens), _ptr(part_o), _ptr(part_ml),
                     _ptr(_split_counters(q.device)), _c_int(blocks), *tail[:-1], *fused, *extra, tail[-1])
        return out
    if raw is not None:
        raise ValueError("raw q, k, v rows are taken by the decode kernel only")
    if tokens > ctx.real_tokens:
        out[ctx.real_tokens:].zero_()
    # The single tokens of a step that also carries prompt portions: the decode kernel over that
    # selection of rows (split keys, every block busy), not one 64-row tile a token and kv head.
    shortest = 0
    if ratio <= 16 and decode_uses_tma(library, head_dim, ratio, page_size):
        rows, row_positions, row_slots, n_single = single_tokens(ctx)
        cluster = decode_cluster(library, head_dim, ratio, page_size, n_single, kv_heads, ctx.max_kv_len) if n_single else 0
        if cluster:
            status = ops.status_word(q.device, "attn_decode_tma", {1: "the TMA producer", 2: "the consumer warps"})
            library.call("mrun_attn_decode_cluster", _ptr(q), _c_long(q_stride), _ptr(out), _ptr(cache.k), _ptr(cache.v),
                         _ptr(group.block_tables), _c_int(group.max_blocks), _ptr(row_slots), _ptr(row_positions),
                         _c_int(n_single), _c_int(cluster), *tail[:-1],
                         _c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None),
                         _ptr(rows), _c_long(pages), _ptr(status), tail[-1])
            shortest = 1
        elif n_single and n_single * kv_heads <= COUNTER_CAPACITY:
            blocks, splits = decode_launch(n_single, kv_heads, decode_slots(head_dim, ratio, page_size))
            part_o = torch.empty((blocks, 2, 16, head_dim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((blocks, 2, 16, 2), dtype=torch.float32, device=q.device)
            prefix, assignment = decode_plan(ctx, library, window, kv_heads, blocks, splits, positions=row_positions)
            status = ops.status_word(q.device, "attn_decode_tma", {1: "the TMA producer", 2: "the consumer warps"})
            library.call("mrun_attn_decode_tma", _ptr(q), _c_long(q_stride), _ptr(out), _ptr(cache.k), _ptr(cache.v),
                         _ptr(group.block_tables), _c_int(group.max_blocks), _ptr(row_slots), _ptr(row_positions),
                         _ptr(prefix), _ptr(assignment), _c_int(n_single), _ptr(part_o), _ptr(part_ml),
                         _ptr(_split_counters(q.device)), _c_int(blocks), *tail[:-1],
                         _c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None),
                         _ptr(rows), _c_long(pages), _ptr(status), tail[-1])
            shortest = 1
    short_up_to = 1 << 30
    if prefill_uses_tcgen05(library, head_dim, ratio, page_size):
        # segments with more rows than a 64-row tile go to the 128-row tcgen05 kernel
        short_up_to = (64 // ratio) if ratio <= 64 else 0
        first, count, n_tiles = prefill_tiles(ctx, 128 // ratio, longer_than=max(short_up_to, shortest))
        if n_tiles:
            status = ops.status_word(q.device, "attn_prefill_tc5",
                                     {1: "a key/value loader", 2: "the MMA issuer", 3: "the softmax warps"})
            library.call("mrun_attn_prefill_tc5", _ptr(q), _c_long(q_stride), _ptr(out), *common, _ptr(first),
                         _ptr(count), _c_int(n_tiles), *tail[:-1], _c_long(pages), _ptr(status), tail[-1])
    if short_up_to > shortest:
        first, count, n_tiles = prefill_tiles(ctx, 64 // ratio, longer_than=shortest, up_to=short_up_to)
        if n_tiles:
            library.call("mrun_attn_prefill", _ptr(q), _c_long(q_stride), _ptr(out), *common, _ptr(first),
                         _ptr(count), _c_int(n_tiles), *tail)
    return out


TC5_PREFILL = True       # False: the mma.sync kernel for every prompt portion (tests compare the two)
_tc5_prefill = {}


def prefill_uses_tcgen05(library, head_dim: int, ratio: int, page_size: int) -> bool:
    """Head sizes 64 and 128, pages of a power-of-two size (the kernel copies whole pages by TMA)."""
    if not TC5_PREFILL or ratio > 128 or page_size & (page_size - 1):
        return False
    have = _tc5_prefill.get(head_dim)
    if have is None:
        have = _tc5_prefill[head_dim] = bool(library._dll.mrun_attn_prefill_tc5_available())
    return have
