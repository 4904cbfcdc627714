"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))`` with SiLU
(crates/mrun-engine/src/models/common.rs:312-345, crates/mrun-engine/src/models/activations.rs:46-59).
gate and up run as one product with the weights stacked (this file's own concatenation); with at
most 16 rows the activation is applied in that product's epilogue."""
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
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        # bfloat16: gate and up rows interleaved in runs of eight, so that the decode GEMM's
        # epilogue finds a gate and its up in one thread and applies the activation itself
        self.interleaved = runtime.precision.act == torch.bfloat16 and spec.intermediate % 8 == 0
        if self.interleaved:
            stacked = torch.stack([gate.view(-1, 8, spec.hidden), up.view(-1, 8, spec.hidden)], dim=1)
            self.w_gate_up = runtime.matrix(stacked.reshape(2 * spec.intermediate, spec.hidden))
        else:
            self.w_gate_up = runtime.matrix(torch.cat([gate, up], dim=0))
        self.w_down = runtime.matrix(tensors["down_proj.weight"])

    def activation_elements(self) -> int:
        """Elements per token of the temporaries alive at once (gate, up and their product)."""
        return 3 * self.spec.intermediate

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if self.interleaved and ops.skinny_ok(x, self.w_gate_up):
            act = ops.gemm_skinny(x, self.w_gate_up, swiglu_rows=True)
        elif self.interleaved and ops.tc5_ok(x, self.w_gate_up):
            act = ops.gemm_tc5(x, self.w_gate_up, swiglu_rows=True)
        else:
            gate_up = ops.linear(x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.spec.intermediate), dtype=x.dtype, device=x.device)
            ops.swiglu(gate_up, act, interleaved=self.interleaved)
        return ops.linear(act, self.w_down)
