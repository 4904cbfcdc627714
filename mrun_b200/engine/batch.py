"""The description of one step that the parts and kernels read.

A step is a flat batch of tokens cut into *segments*: one per request, each a run of consecutive
tokens of that request (a portion of its prompt, or one decoded token).  Everything a kernel needs
is in int32 device arrays built on the host in one pinned buffer and copied once.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import FREED, CacheManager, RequestCache


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""

    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class SegmentInfo:
    slot: int          # the request's state slot
    q_start: int       # first row of the segment in the flat batch
    q_len: int
    pos_start: int     # position of its first token = tokens the request already holds


@dataclass
class GroupView:
    """A cache group's view of the step."""

    block_tables: torch.Tensor   # int32 [segments, max_blocks], FREED where no page is held
    slot_mapping: torch.Tensor   # int32 [tokens]: page * page_size + offset of each new token
    max_blocks: int


@dataclass
class StepContext:
    num_tokens: int
    num_segments: int
    segments: List[SegmentInfo]
    token_ids: torch.Tensor      # int32 [tokens]
    positions: torch.Tensor      # int32 [tokens]; negative = padding row
    token_seg: torch.Tensor      # int32 [tokens]: segment of each token
    seg_q_start: torch.Tensor    # int32 [segments + 1]
    seg_kv_len: torch.Tensor     # int32 [segments]: keys visible to the segment's last token
    seg_slot: torch.Tensor       # int32 [segments]
    groups: Dict[tuple, GroupView]
    max_q_len: int
    max_kv_len: int
    page_size: int
    shared: dict = field(default_factory=dict)   # per-step results shared between layers

    def group(self, key: tuple) -> GroupView:
        return self.groups[key]

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


class HostStaging:
    """Two pinned buffers used in turn; a buffer is reused only after its copy has finished."""

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: List[Optional[torch.Tensor]] = [None, None]
        self._events: List[Optional[torch.cuda.Event]] = [None, None]
        self._turn = 0

    def upload(self, host: np.ndarray) -> torch.Tensor:
        i = self._turn
        self._turn ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()
        n = host.size
        if self._buffers[i] is None or self._buffers[i].numel() < n:
            self._buffers[i] = torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True)
        pinned = self._buffers[i][:n]
        pinned.numpy()[:] = host
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        out.copy_(pinned, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._events[i] = event
        return out


def build_context(entries: Sequence[StepEntry], manager: CacheManager, staging: HostStaging) -> StepContext:
    """Lays the step out.  The requests' pages for the new tokens are already planned
    (``request.pending`` tokens, blocks extended)."""
    page_size = manager.page_size
    n_seg = len(entries)
    lengths = [len(e.tokens) for e in entries]
    total = sum(lengths)
    keys = list(manager.groups)
    max_blocks = max(1, max(len(e.request.blocks[k]) for e in entries for k in keys) if keys else 1)

    per_group = total + n_seg * max_blocks
    host = np.empty(3 * total + (n_seg + 1) + 2 * n_seg + len(keys) * per_group, dtype=np.int32)
    token_ids, positions, token_seg = host[:total], host[total:2 * total], host[2 * total:3 * total]
    at = 3 * total
    seg_q_start = host[at:at + n_seg + 1]; at += n_seg + 1
    seg_kv_len = host[at:at + n_seg]; at += n_seg
    seg_slot = host[at:at + n_seg]; at += n_seg
    group_off = at

    segments: List[SegmentInfo] = []
    row = 0
    for s, entry in enumerate(entries):
        n, start = lengths[s], entry.request.length
        token_ids[row:row + n] = np.asarray(entry.tokens, dtype=np.int64)
        positions[row:row + n] = np.arange(start, start + n, dtype=np.int32)
        token_seg[row:row + n] = s
        seg_q_start[s] = row
        seg_kv_len[s] = start + n
        seg_slot[s] = entry.request.slot
        segments.append(SegmentInfo(entry.request.slot, row, n, start))
        row += n
    seg_q_start[n_seg] = total

    for g, key in enumerate(keys):
        base = group_off + g * per_group
        slot_mapping = host[base:base + total]
        tables = host[base + total:base + per_group].reshape(n_seg, max_blocks)
        tables[:] = FREED
        for s, entry in enumerate(entries):
            blocks = np.asarray(entry.request.blocks[key], dtype=np.int32)
            tables[s, :len(blocks)] = blocks
            pos = positions[seg_q_start[s]:seg_q_start[s + 1]]
            pages = blocks[pos // page_size]
            slot_mapping[seg_q_start[s]:seg_q_start[s + 1]] = np.where(
                pages == FREED, -1, pages * page_size + pos % page_size)

    dev = staging.upload(host)
    groups = {}
    for g, key in enumerate(keys):
        base = group_off + g * per_group
        groups[key] = GroupView(dev[base + total:base + per_group].view(n_seg, max_blocks),
                                dev[base:base + total], max_blocks)
    at = 3 * total
    return StepContext(
        num_tokens=total, num_segments=n_seg, segments=segments,
        token_ids=dev[:total], positions=dev[total:2 * total], token_seg=dev[2 * total:3 * total],
        seg_q_start=dev[at:at + n_seg + 1], seg_kv_len=dev[at + n_seg + 1:at + 2 * n_seg + 1],
        seg_slot=dev[at + 2 * n_seg + 1:at + 3 * n_seg + 1], groups=groups,
        max_q_len=max(lengths), max_kv_len=int(seg_kv_len.max()), page_size=page_size)
