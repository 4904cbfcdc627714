"""The description of one step that the parts and kernels read.

A step is a flat batch of tokens cut into *segments*: one per request, each a run of consecutive
tokens of that request (a portion of its prompt, or one decoded token).  Everything a kernel needs
is in int32 device arrays that the host lays out in one pinned buffer and copies once.  The block
tables live on the device, one row per state slot, and only their changes travel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import FREED, CacheManager, RequestCache
from ..kernels import ops


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

    block_tables: torch.Tensor   # int32 [state slots, max_blocks], FREED where no page is held
    slot_mapping: torch.Tensor   # int32 [tokens]: page * page_size + offset of each new token, -1 = none
    max_blocks: int


@dataclass
class StepContext:
    num_tokens: int              # rows of the batch, padding rows included
    num_segments: int
    segments: List[SegmentInfo]
    token_ids: torch.Tensor      # int32 [tokens]
    positions: torch.Tensor      # int32 [tokens]; negative = padding row
    token_slot: torch.Tensor     # int32 [tokens]: state slot (block-table row) of each token
    seg_q_start: torch.Tensor    # int32 [segments + 1]
    seg_kv_len: torch.Tensor     # int32 [segments]: keys visible to the segment's last token
    seg_slot: torch.Tensor       # int32 [segments]
    groups: Dict[tuple, GroupView]
    max_q_len: int
    max_kv_len: int
    page_size: int
    real_tokens: int = 0         # rows that are not padding
    upload: Optional[object] = None              # host int32 array -> device tensor (pinned staging)
    shared: dict = field(default_factory=dict)   # per-step results shared between layers

    def group(self, key: tuple) -> GroupView:
        return self.groups[key]

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


class HostStaging:
    """Pinned buffers used in turn; a buffer is reused only after its copy has finished."""

    def __init__(self, device: torch.device, depth: int = 4):
        self.device = device
        self._buffers: List[Optional[torch.Tensor]] = [None] * depth
        self._events: List[Optional[torch.cuda.Event]] = [None] * depth
        self._turn = 0
        self.bytes_uploaded = 0

    def upload(self, host: np.ndarray, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        i = self._turn
        self._turn = (self._turn + 1) % len(self._buffers)
        if self._events[i] is not None:
            self._events[i].synchronize()
        n = host.size
        if self._buffers[i] is None or self._buffers[i].numel() < n:
            self._buffers[i] = torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True)
        pinned = self._buffers[i][:n]
        pinned.numpy()[:] = host
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=self.device)
        out[:n].copy_(pinned, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._events[i] = event
        self.bytes_uploaded += 4 * n
        return out


RECENT = 20   # token ids per row that the repetition penalty looks at


def layout(tokens: int, segments: int, groups: int, sampling_rows: int = 0) -> Dict[str, slice]:
    """Where each array sits in the step's int32 buffer.  With ``sampling_rows`` the buffer also
    carries, per row, where its token comes from (``token_src``: a row of the previous captured
    step, or -1 for the id the host wrote) and the sampling settings (floats as their bit
    patterns, 64-bit keys as pairs on an even offset)."""
    names = [("token_ids", tokens), ("positions", tokens), ("token_slot", tokens),
             ("seg_q_start", segments + 1), ("seg_kv_len", segments), ("seg_slot", segments)]
    names += [(f"slot_mapping{g}", tokens) for g in range(groups)]
    if sampling_rows:
        r = sampling_rows
        names += [("token_src", r), ("temperature", r), ("top_p", r), ("min_p", r), ("penalty", r), ("top_k", r),
                  ("recent", RECENT * r), ("keys", 2 * r)]
    out, at = {}, 0
    for name, n in names:
        if name == "keys":
            at += at % 2
        out[name] = slice(at, at + n)
        at += n
    out["_size"] = slice(0, at)
    return out


def push_table_updates(manager: CacheManager, staging: HostStaging) -> None:
    """Brings the device block tables up to date with what the host handed out or took back."""
    for key, (index, value) in manager.drain_table_updates().items():
        both = staging.upload(np.concatenate([index, value]))
        n = index.size
        ops.scatter_i32(manager.groups[key].table_device, both[:n], both[n:])


def build_context(entries: Sequence[StepEntry], manager: CacheManager, staging: HostStaging,
                  pad_tokens: Optional[int] = None, out: Optional[torch.Tensor] = None,
                  sampling=None) -> StepContext:
    """Lays the step out.  The requests' pages for the new tokens are already planned
    (``request.pending`` tokens, blocks extended).  ``pad_tokens`` appends padding rows
    (position -1, no cache slot) up to that many rows and pads the segment arrays to the same
    count, for steps that replay a captured graph of fixed shape; ``out`` is the graph's own
    buffer to fill, and ``sampling(host, where)`` fills the sampling settings it also carries."""
    page_size = manager.page_size
    lengths = [len(e.tokens) for e in entries]
    real = sum(lengths)
    total = max(real, pad_tokens or 0)
    n_seg = len(entries) if pad_tokens is None else pad_tokens
    keys = list(manager.groups)
    where = layout(total, n_seg, len(keys), total if sampling is not None else 0)
    host = np.zeros(where["_size"].stop, dtype=np.int32)
    if sampling is not None:
        host[where["token_src"]] = -1
        sampling(host, where)
    token_ids, positions, token_slot = host[where["token_ids"]], host[where["positions"]], host[where["token_slot"]]
    seg_q_start, seg_kv_len, seg_slot = host[where["seg_q_start"]], host[where["seg_kv_len"]], host[where["seg_slot"]]
    positions[real:] = -1
    maps = [host[where[f"slot_mapping{g}"]] for g in range(len(keys))]
    for m in maps:
        m[real:] = -1

    # positions, slots, segment bounds and every token's place in the pages: the native books know them
    slots = [e.request.slot for e in entries]
    manager.layout_step(slots, lengths, positions, token_slot, seg_q_start, seg_kv_len, seg_slot, maps)
    if max(lengths) == 1:
        token_ids[:len(entries)] = [e.tokens[0] for e in entries]
    else:
        token_ids[:real] = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
    starts = seg_kv_len[:len(entries)] - np.asarray(lengths, dtype=np.int32)
    segments = [SegmentInfo(slot, int(q0), n, int(p))
                for slot, q0, n, p in zip(slots, seg_q_start[:len(entries)].tolist(), lengths, starts.tolist())]
    seg_q_start[len(entries):] = real

    push_table_updates(manager, staging)
    dev = staging.upload(host, out)
    groups = {key: GroupView(manager.groups[key].table_device, dev[where[f"slot_mapping{g}"]],
                             manager.groups[key].max_blocks)
              for g, key in enumerate(keys)}
    return StepContext(
        num_tokens=total, num_segments=n_seg, segments=segments,
        token_ids=dev[where["token_ids"]], positions=dev[where["positions"]],
        token_slot=dev[where["token_slot"]], seg_q_start=dev[where["seg_q_start"]],
        seg_kv_len=dev[where["seg_kv_len"]], seg_slot=dev[where["seg_slot"]], groups=groups,
        max_q_len=max(lengths), max_kv_len=int(seg_kv_len.max()), page_size=page_size,
        real_tokens=real, upload=staging.upload)
