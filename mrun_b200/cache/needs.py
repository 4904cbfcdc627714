"""What a mixer asks of the cache manager.

A mixer declares one *need* (or none).  Needs with the same ``group_key`` share a page pool and a
block table per request; each schedule entry still has tensors of its own inside the group.
The reference draws the same line per layer between key/value state that grows with the
sequence and recurrent state of fixed size (``LayerState::{Kv, Recurrent}``,
crates/mrun-engine/src/state.rs:87-117).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token (``window`` None) or of the last ``window`` tokens."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> tuple:
        return ("paged", self.window)


@dataclass(frozen=True)
class FixedState:
    """Per-request state of a fixed shape, zero when a request starts."""

    shape: Tuple[int, ...]
    dtype: str = "float32"

    def group_key(self) -> tuple:
        return ("state",)
