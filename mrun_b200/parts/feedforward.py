"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``, act = SiLU for Qwen3
(crates/mrun-engine/src/models/common.rs:312-345, crates/mrun-engine/src/models/activations.rs:46-59).
gate and up run as one product with the weights stacked (this file's own concatenation); with at
most 16 rows the activation is applied in that product's epilogue.  The gate's function is a name
the kernels know by a code (``ops.GATE_FUNCTIONS``); a projection's ``.bias`` is bound and added
when the checkpoint has one (crates/mrun-engine/src/load.rs:281,302-305)."""
from __future__ import annotations

import torch

from ..config.spec import GatedMLPSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP:
    accepts_normed_rows = True      # its first product takes ``ops.NormedRows`` as x
    can_defer_output = True         # ``forward(..., defer_output=True)`` may return ``ops.PendingLinear``
    @staticmethod
    def tensor_specs(spec: GatedMLPSpec, prefix: str):
        return [
            TensorSpec(f"{prefix}.gate_proj.weight", (spec.intermediate, spec.hidden)),
            TensorSpec(f"{prefix}.up_proj.weight", (spec.intermediate, spec.hidden)),
            TensorSpec(f"{prefix}.down_proj.weight", (spec.hidden, spec.intermediate)),
            TensorSpec(f"{prefix}.gate_proj.bias", (spec.intermediate,), optional=True),
            TensorSpec(f"{prefix}.up_proj.bias", (spec.intermediate,), optional=True),
            TensorSpec(f"{prefix}.down_proj.bias", (spec.hidden,), optional=True),
        ]

    def __init__(self, spec: GatedMLPSpec, tensors, runtime: Runtime):
        ops.gate_code(spec.activation)       # refuses a gate function no kernel has
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
        self.b_gate_up = None
        gate_bias, up_bias = tensors.get("gate_proj.bias"), tensors.get("up_proj.bias")
        if gate_bias is not None or up_bias is not None:
            zeros = torch.zeros(spec.intermediate, dtype=torch.float32)
            gate_bias = zeros if gate_bias is None else gate_bias.to(torch.float32)
            up_bias = zeros if up_bias is None else up_bias.to(torch.float32)
            if self.interleaved:
                both = torch.stack([gate_bias.view(-1, 8), up_bias.view(-1, 8)], dim=1).reshape(-1)
            else:
                both = torch.cat([gate_bias, up_bias])
            self.b_gate_up = runtime.vector_f32(both)
        self.b_down = runtime.vector_f32(tensors["down_proj.bias"]) if "down_proj.bias" in tensors else None

    def activation_elements(self) -> int:
        """Elements per token of the temporaries alive at once (gate, up and their product)."""
        return 3 * self.spec.intermediate

    def forward(self, x, ctx, defer_output: bool = False):
        name = self.spec.activation
        if self.interleaved and self.b_gate_up is None and ops.skinny_ok(x, self.w_gate_up):
            act = ops.gemm_skinny(x, self.w_gate_up, swiglu_rows=True, activation=name)
        elif self.interleaved and self.b_gate_up is None and ops.tc5_ok(x, self.w_gate_up):
            act = ops.gemm_tc5(x, self.w_gate_up, swiglu_rows=True, activation=name)
        else:
            gate_up = ops.linear(x, self.w_gate_up, bias=self.b_gate_up)
            act = torch.empty((gate_up.shape[0], self.spec.intermediate), dtype=gate_up.dtype, device=gate_up.device)
            ops.swiglu(gate_up, act, interleaved=self.interleaved, activation=name)
        if defer_output:
            return ops.linear_or_pending(act, self.w_down, self.b_down)
        return ops.linear(act, self.w_down, bias=self.b_down)
