"""Architecture-neutral description of a decoder: what the parts are and how they are arranged.

A model is data: a tuple of :class:`LayerSpec` (which mixer, which feed-forward, which norms, under
which tensor-name prefixes) and a *schedule*, the order in which layers run.  A schedule entry may
name a layer that an earlier entry already named (the layer's weights run twice, each run with a
cache of its own) or read the cache that an earlier entry wrote (``cache_of``).  Every part spec
carries its own sizes and constants; nothing below this file knows which architecture it serves.

The reference keeps the same split between a layer's parts and their constants
(``Layer{input_layernorm, attention, post_attention_layernorm, mlp}``,
crates/mrun-engine/src/models/qwen3.rs:16-21; ``AttentionConfig``,
crates/mrun-engine/src/models/common.rs:50-64) and a per-layer kind list that drives the state
layout (crates/mrun-engine/src/models/registry.rs:208-247).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, ClassVar, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part expects in the checkpoint.

    ``init`` tells the random-weights mode how to fill it: ``"normal"`` (matrices and tables),
    ``"norm"`` (scale vectors: ones, or ones plus noise).  An ``optional`` tensor is bound when
    the checkpoint has it and is neither missed nor made by the random-weights mode otherwise
    (the reference takes a linear layer's ``.bias`` that way, crates/mrun-engine/src/load.rs:281).
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False


# --------------------------------------------------------------------------- norms

@dataclass(frozen=True)
class RMSNormSpec:
    kind: ClassVar[str] = "rmsnorm"
    size: int
    eps: float


# --------------------------------------------------------------------------- position encodings

@dataclass(frozen=True)
class RotarySpec:
    """Rotary positions, half-split pairing: feature j pairs with j + rotary_dim/2."""

    kind: ClassVar[str] = "rotary"
    head_dim: int
    rotary_dim: int
    theta: float


# --------------------------------------------------------------------------- mixers

@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` = None: a token sees every earlier key.  ``window`` = W: it sees the last W keys,
    itself included.
    """

    kind: ClassVar[str] = "attention"
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    softmax_scale: float
    qk_norm: Optional[RMSNormSpec] = None
    position: Optional[Any] = None
    window: Optional[int] = None


# --------------------------------------------------------------------------- feed-forwards

@dataclass(frozen=True)
class GatedMLPSpec:
    """``down(act(gate(x)) * up(x))``; ``activation`` names the gate's function."""

    kind: ClassVar[str] = "gated_mlp"
    hidden: int
    intermediate: int
    activation: str = "silu"


# --------------------------------------------------------------------------- layers and model

@dataclass(frozen=True)
class LayerSpec:
    """One block: norm → mixer → residual → norm → feed-forward → residual (``pre_norm``)."""

    prefix: str
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    arrangement: str = "pre_norm"
    mixer_prefix: str = "self_attn"
    feed_forward_prefix: str = "mlp"
    mixer_norm_prefix: str = "input_layernorm"
    feed_forward_norm_prefix: str = "post_attention_layernorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` = index of an *earlier schedule entry* whose cache this
    run reads instead of owning one (it then writes nothing into it)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    final_norm: Any
    tie_embeddings: bool
    schedule: Tuple[ScheduleEntry, ...] = ()
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm"
    head_name: str = "lm_head.weight"
    eos_token_ids: Tuple[int, ...] = ()
    # optional transform specs (kinds of the ``TRANSFORMS`` registry; a spec that binds tensors
    # carries their ``prefix``): applied to the 32-bit stream right after the embedding, and to
    # the float32 logits of the wanted rows
    embedding_transform: Any = None
    logits_transform: Any = None
    # tensors that may be present in a checkpoint and are dropped unread: the vision tower, heads
    # for multi-token prediction and rotary frequency tables
    # (crates/mrun-engine/src/load.rs:168-173, crates/mrun-engine/src/models/qwen3.rs:107)
    ignored_suffixes: Tuple[str, ...] = ()
    ignored_prefixes: Tuple[str, ...] = ("vision_tower", "model.visual")
    ignored_containing: Tuple[str, ...] = ("mtp.", "rotary_emb.inv_freq")
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    def ignores(self, name: str) -> bool:
        """Whether a checkpoint tensor of this name is left unread."""
        return (name.startswith(tuple(self.ignored_prefixes)) or name.endswith(tuple(self.ignored_suffixes))
                or any(part in name for part in self.ignored_containing))

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i) for i in range(len(self.layers)))

    def validate(self) -> None:
        order = self.run_order()
        for at, entry in enumerate(order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {at} names layer {entry.layer}, "
                                 f"the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < at:
                    raise ValueError(f"schedule entry {at} reads the cache of entry "
                                     f"{entry.cache_of}, which does not run before it")
                if order[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {at} reads the cache of entry "
                                     f"{entry.cache_of}, which owns none")
