"""Rotary position encoding, half-split pairing.

For pair j of a head (features j and j + rotary_dim/2) at position p: angle = p * theta^(-2j/rotary_dim),
``(y_j, y_{j+half}) = (x_j cos - x_{j+half} sin, x_{j+half} cos + x_j sin)``
(crates/mrun-engine/src/models/common.rs:215-230, 264-280).  The part only produces the table of
(cos, sin) per token and pair, once per step; the attention's fused kernel applies it.
"""
from __future__ import annotations

import torch

from ..config.spec import RotarySpec
from ..kernels import ops
from .base import Runtime, register_position


@register_position("rotary")
class Rotary:
    @staticmethod
    def tensor_specs(spec: RotarySpec, prefix: str):
        return []

    def __init__(self, spec: RotarySpec, tensors, runtime: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim must be even and in (0, head_dim={spec.head_dim}], got {spec.rotary_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        half = spec.rotary_dim // 2
        exponents = torch.arange(half, dtype=torch.float64) * (-2.0 / spec.rotary_dim)
        self.inv_freq = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), exponents).to(runtime.device)

    def rotation(self, ctx) -> torch.Tensor:
        key = ("rotary", self.spec)
        table = ctx.shared.get(key)
        if table is None:
            table = torch.empty((ctx.num_tokens, self.rotary_dim // 2, 2), dtype=torch.float32,
                                device=self.inv_freq.device)
            ops.rotary_table(ctx.positions, self.inv_freq, table)
            ctx.shared[key] = table
        return table
