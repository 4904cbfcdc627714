"""The pre-norm arrangement of a layer: ``x += mixer(norm(x)); x += ff(norm(x))``
(crates/mrun-engine/src/models/qwen3.rs:133-145).

The residual sum is fused with the norm that follows it: a block receives the 32-bit stream and the
previous branch's output that has not been added yet, and returns its own feed-forward output
unadded.  The sum itself is 32-bit.

Two optional capabilities let a decode step fold that sum and norm into the products around
them; a part that does not declare them gets and gives plain tensors.  A mixer or feed-forward
with ``can_defer_output`` may return its last product unrun (``ops.PendingLinear``) when called
with ``defer_output=True``; a norm with ``accepts_pending`` takes it as ``delta`` and may answer
with ``ops.NormedRows``; a part with ``accepts_normed_rows`` takes those as its ``x``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec, TensorSpec
from ..kernels import ops
from .base import FEED_FORWARDS, MIXERS, NORMS, Runtime, local, register_arrangement


def norm_add(norm, resid: torch.Tensor, delta):
    """``norm.add_forward`` for a ``delta`` that may be pending: computed first unless the norm
    takes it as it is."""
    if isinstance(delta, ops.PendingLinear) and not getattr(norm, "accepts_pending", False):
        delta = delta.compute()
    return norm.add_forward(resid, delta)


def part_input(part, h):
    """Normed rows for a part: finished into a plain tensor unless the part takes them as they are."""
    if isinstance(h, ops.NormedRows) and not getattr(part, "accepts_normed_rows", False):
        h = h.finish()
    return h


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
        self._mixer_defers = bool(getattr(self.mixer, "can_defer_output", False))
        self._feed_forward_defers = bool(getattr(self.feed_forward, "can_defer_output", False))

    accepts_pending = True      # ``delta`` may be an ``ops.PendingLinear``, and so may the result

    def forward(self, resid: torch.Tensor, delta, ctx, cache):
        h = part_input(self.mixer, norm_add(self.mixer_norm, resid, delta))
        if self._mixer_defers:
            a = self.mixer.forward(h, ctx, cache, defer_output=True)
        else:
            a = self.mixer.forward(h, ctx, cache)
        h = part_input(self.feed_forward, norm_add(self.feed_forward_norm, resid, a))
        if self._feed_forward_defers:
            return self.feed_forward.forward(h, ctx, defer_output=True)
        return self.feed_forward.forward(h, ctx)
