"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))`` with SiLU
(crates/mrun-engine/src/models/common.rs:312-345, crates/mrun-engine/src/models/activations.rs:46-59).
gate and up run as one product with the weights stacked (this file's own concatenation)."""
from __future__ import annotations

import torch

from ..config.spec import GatedMLPSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP:
    @staticmethod
    def tensor_specs(spec: GatedMLPSpec, prefix: str):
        return [
            TensorSpec(f"{prefix}.gate_proj.weight", (spec.intermediate, spec.hidden)),
            TensorSpec(f"{prefix}.up_proj.weight", (spec.intermediate, spec.hidden)),
            TensorSpec(f"{prefix}.down_proj.weight", (spec.hidden, spec.intermediate)),
        ]

    def __init__(self, spec: GatedMLPSpec, tensors, runtime: Runtime):
        if spec.activation != "silu":
            raise ValueError(f"the gated feed-forward has a kernel for silu only, got {spec.activation!r}")
        self.spec = spec
        self.w_gate_up = runtime.matrix(torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0))
        self.w_down = runtime.matrix(tensors["down_proj.weight"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        gate_up = ops.linear(x, self.w_gate_up)
        act = torch.empty((x.shape[0], self.spec.intermediate), dtype=x.dtype, device=x.device)
        ops.swiglu(gate_up, act)
        return ops.linear(act, self.w_down)
