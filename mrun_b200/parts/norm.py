"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * w`` in 32-bit
(crates/mrun-engine/src/load.rs:348-364; the form with eps added to the mean is stated at
crates/mrun-engine/src/models/gated_delta.rs:11-13)."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import RMSNormSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def tensor_specs(spec: RMSNormSpec, prefix: str):
        return [TensorSpec(f"{prefix}.weight", (spec.size,), "norm")]

    # ``delta`` may be a product that has not run yet (``ops.PendingLinear``): with a handful
    # of rows it runs with the residual sum and this norm folded into its epilogue, and what
    # comes back is ``ops.NormedRows`` (the row scale is applied by the product that reads it);
    # with more rows the vendor GEMM adds it into the 32-bit stream itself.
    accepts_pending = True

    def __init__(self, spec: RMSNormSpec, tensors, runtime: Runtime):
        self.size, self.eps = spec.size, float(spec.eps)
        self.weight = runtime.vector_f32(tensors["weight"])
        self.act = runtime.precision.act

    def add_forward(self, resid: torch.Tensor, delta):
        if isinstance(delta, ops.PendingLinear):
            if ops.norm_fusable(delta, resid, self.weight):
                return ops.linear_into_norm(delta, resid, self.weight, self.eps)
            if ops.accumulate_ok(delta, resid):
                ops.linear_add_into(resid, delta)          # the sum rides in the vendor GEMM
                delta = None
            else:
                delta = delta.compute()
        out = torch.empty(resid.shape, dtype=self.act, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)

    def rows_forward(self, resid: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        if isinstance(delta, ops.PendingLinear):
            delta = delta.compute()
        out = torch.empty((rows.numel(), self.size), dtype=self.act, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows=rows)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_forward(x.to(torch.float32), None)
