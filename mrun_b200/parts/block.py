"""The pre-norm arrangement of a layer: ``x += mixer(norm(x)); x += ff(norm(x))``
(crates/mrun-engine/src/models/qwen3.rs:133-145).

The residual sum is fused with the norm that follows it: a block receives the 32-bit stream and the
previous branch's output that has not been added yet, and returns its own feed-forward output
unadded.  The sum itself is 32-bit.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec, TensorSpec
from .base import FEED_FORWARDS, MIXERS, NORMS, Runtime, local, register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str = "") -> list[TensorSpec]:
        p = spec.prefix
        return (NORMS.tensor_specs(spec.mixer_norm, f"{p}.{spec.mixer_norm_prefix}")
                + MIXERS.tensor_specs(spec.mixer, f"{p}.{spec.mixer_prefix}")
                + NORMS.tensor_specs(spec.feed_forward_norm, f"{p}.{spec.feed_forward_norm_prefix}")
                + FEED_FORWARDS.tensor_specs(spec.feed_forward, f"{p}.{spec.feed_forward_prefix}"))

    def __init__(self, spec: LayerSpec, tensors, runtime: Runtime):
        mine = local(tensors, spec.prefix)
        self.mixer_norm = NORMS.build(spec.mixer_norm, local(mine, spec.mixer_norm_prefix), runtime)
        self.mixer = MIXERS.build(spec.mixer, local(mine, spec.mixer_prefix), runtime)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, local(mine, spec.feed_forward_norm_prefix), runtime)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, local(mine, spec.feed_forward_prefix), runtime)

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        h = self.mixer_norm.add_forward(resid, delta)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.add_forward(resid, a)
        return self.feed_forward.forward(h, ctx)
