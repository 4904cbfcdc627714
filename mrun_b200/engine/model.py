"""A decoder assembled from a :class:`ModelSpec`: embedding, the scheduled runs of its layers, the
final norm and the output head at the wanted rows.

The model is the same object whatever the architecture; which parts it holds and in which order
they run comes from the spec (reference: ``embed`` → every ``layer`` → ``logits`` on the last row,
crates/mrun-engine/src/nuvec_engine.rs:999-1028, crates/mrun-engine/src/models/common.rs:382-414).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from ..parts import ARRANGEMENTS, NORMS, TRANSFORMS, Runtime
from ..parts.base import local
from .batch import StepContext


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = runtime.matrix(tensors[spec.embedding_name])
        if self.embedding.shape != (spec.vocab_size, spec.hidden_size):
            raise ValueError("the embedding table does not have the spec's shape")
        self.head = self.embedding if spec.tie_embeddings else runtime.matrix(tensors[spec.head_name])
        self.blocks = [ARRANGEMENTS.get(layer.arrangement)(layer, tensors, runtime) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, local(tensors, spec.final_norm_prefix), runtime)
        self.order = spec.run_order()
        self.embedding_transform = self.logits_transform = None
        if spec.embedding_transform is not None:
            t = spec.embedding_transform
            self.embedding_transform = TRANSFORMS.build(t, local(tensors, getattr(t, "prefix", "")), runtime)
        if spec.logits_transform is not None:
            t = spec.logits_transform
            self.logits_transform = TRANSFORMS.build(t, local(tensors, getattr(t, "prefix", "")), runtime)

    # ------------------------------------------------------------------ cache layout
    def cache_needs(self) -> List[object]:
        """The need of each schedule entry (None for entries that read another's cache)."""
        needs = []
        for entry in self.order:
            mixer = self.blocks[entry.layer].mixer
            needs.append(None if entry.cache_of is not None else mixer.cache_need())
        return needs

    def cache_shares(self) -> List[Optional[int]]:
        return [entry.cache_of for entry in self.order]

    def activation_elements(self) -> int:
        """The widest set of per-token temporaries any part declares (parts without the hint
        count as nothing); the memory budget sizes the step's scratch from it."""
        widest = 0
        for block in self.blocks:
            for part in (getattr(block, "mixer", None), getattr(block, "feed_forward", None)):
                hint = getattr(part, "activation_elements", None)
                if hint is not None:
                    widest = max(widest, int(hint()))
        return widest

    @property
    def graph_safe(self) -> bool:
        return all(getattr(block.mixer, "graph_safe", False) for block in self.blocks)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def walk(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif hasattr(obj, "__dict__"):
                for value in vars(obj).values():
                    if isinstance(value, (torch.Tensor,)) or hasattr(value, "__dict__"):
                        walk(value)
                    elif isinstance(value, (list, tuple)):
                        for item in value:
                            walk(item)
        walk(self.final_norm)
        for block in self.blocks:
            walk(block)
        for t in (self.embedding, self.head):
            walk(t)
        return total

    # ------------------------------------------------------------------ forward
    def hidden_states(self, ctx: StepContext, caches) -> tuple:
        """Runs the layers; returns the 32-bit stream and the last branch output not yet added."""
        ops.RowSums.begin_step(self.runtime.device)
        resid = torch.empty((ctx.num_tokens, self.spec.hidden_size), dtype=torch.float32,
                            device=self.runtime.device)
        ops.embed(self.embedding, ctx.token_ids, resid)
        if self.embedding_transform is not None:
            resid = self.embedding_transform.forward(resid)
        delta = None
        for at, entry in enumerate(self.order):
            block = self.blocks[entry.layer]
            if isinstance(delta, ops.PendingLinear) and not getattr(block, "accepts_pending", False):
                delta = delta.compute()
            delta = block.forward(resid, delta, ctx, caches[at])
        return resid, delta

    def logits(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """float32 ``[len(rows), vocab]``: final norm and head at the wanted rows only."""
        if isinstance(delta, ops.PendingLinear):
            delta = delta.compute()
        h = self.final_norm.rows_forward(resid, delta, rows)
        logits = ops.linear(h, self.head, out_dtype=torch.float32)
        if self.logits_transform is not None:
            logits = self.logits_transform.forward(logits)
        return logits

    def forward(self, ctx: StepContext, caches, rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        resid, delta = self.hidden_states(ctx, caches)
        if rows is None or rows.numel() == 0:
            return None
        return self.logits(resid, delta, rows)
