"""Grouped-query attention over the paged cache.

``q, k, v = x Wq^T, x Wk^T, x Wv^T`` as one product with the three weights stacked (this file's own
concatenation; the reference keeps three products, crates/mrun-engine/src/models/common.rs:165-171);
per-head RMSNorm of q and k, then rotation, then k and v into the pages
(crates/mrun-engine/src/models/common.rs:183,194-198); softmax attention of each token over the
keys of its request up to itself; output projection (crates/mrun-engine/src/models/common.rs:137,206).
A projection's ``.bias`` is bound and added when the checkpoint has one
(crates/mrun-engine/src/load.rs:281,302-305); Qwen3's have none.
"""
from __future__ import annotations

import torch

from ..cache.needs import PagedKV
from ..config.spec import AttentionSpec, TensorSpec
from ..kernels import ops
from ..kernels.attention import decode_fuses_input, paged_attention, supports_tensor_cores
from .base import NORMS, POSITIONS, Runtime, register_mixer


@register_mixer("attention")
class Attention:
    accepts_normed_rows = True      # its first product takes ``ops.NormedRows`` as x
    can_defer_output = True         # ``forward(..., defer_output=True)`` may return ``ops.PendingLinear``

    @staticmethod
    def tensor_specs(spec: AttentionSpec, prefix: str):
        d = spec.head_dim
        out = [
            TensorSpec(f"{prefix}.q_proj.weight", (spec.heads * d, spec.hidden)),
            TensorSpec(f"{prefix}.k_proj.weight", (spec.kv_heads * d, spec.hidden)),
            TensorSpec(f"{prefix}.v_proj.weight", (spec.kv_heads * d, spec.hidden)),
            TensorSpec(f"{prefix}.o_proj.weight", (spec.hidden, spec.heads * d)),
            TensorSpec(f"{prefix}.q_proj.bias", (spec.heads * d,), optional=True),
            TensorSpec(f"{prefix}.k_proj.bias", (spec.kv_heads * d,), optional=True),
            TensorSpec(f"{prefix}.v_proj.bias", (spec.kv_heads * d,), optional=True),
            TensorSpec(f"{prefix}.o_proj.bias", (spec.hidden,), optional=True),
        ]
        if spec.qk_norm is not None:
            out += NORMS.tensor_specs(spec.qk_norm, f"{prefix}.q_norm")
            out += NORMS.tensor_specs(spec.qk_norm, f"{prefix}.k_norm")
        if spec.position is not None:
            out += POSITIONS.tensor_specs(spec.position, f"{prefix}.rotary_emb")
        return out

    def __init__(self, spec: AttentionSpec, tensors, runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads={spec.heads} is not a multiple of kv_heads={spec.kv_heads}")
        if spec.qk_norm is not None and spec.qk_norm.size != spec.head_dim:
            raise ValueError("the q/k norm works per head: its size must be head_dim")
        self.spec = spec
        self.runtime = runtime
        self.wqkv = runtime.matrix(torch.cat(
            [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0))
        self.wo = runtime.matrix(tensors["o_proj.weight"])
        biases = [tensors.get(f"{name}_proj.bias") for name in "qkv"]
        self.bqkv = None
        if any(b is not None for b in biases):
            widths = (spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.head_dim)
            self.bqkv = runtime.vector_f32(torch.cat(
                [torch.zeros(n, dtype=torch.float32) if b is None else b.to(torch.float32)
                 for b, n in zip(biases, widths)]))
        self.bo = runtime.vector_f32(tensors["o_proj.bias"]) if "o_proj.bias" in tensors else None
        self.q_weight = self.k_weight = None
        self.eps = 0.0
        if spec.qk_norm is not None:
            self.q_weight = runtime.vector_f32(tensors["q_norm.weight"])
            self.k_weight = runtime.vector_f32(tensors["k_norm.weight"])
            self.eps = float(spec.qk_norm.eps)
        self.position = None
        if spec.position is not None:
            self.position = POSITIONS.build(spec.position, {}, runtime)
        # the tiled kernel that very wide groups fall to needs a tile list made on the host
        ratio = spec.heads // spec.kv_heads
        self.graph_safe = not (supports_tensor_cores(runtime.precision.act, spec.head_dim, ratio) and ratio > 16)

    def cache_need(self):
        return PagedKV(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    def activation_elements(self) -> int:
        """Elements per token of the temporaries alive at once (q, k, v and the heads' output)."""
        return (2 * self.spec.heads + 2 * self.spec.kv_heads) * self.spec.head_dim

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s = self.spec
        group = ctx.group(cache.group_key)
        qkv = ops.linear(x, self.wqkv, bias=self.bqkv)
        rot = self.position.rotation(ctx) if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        slots = group.slot_mapping if cache.writable else None
        out = torch.empty((x.shape[0], s.heads * s.head_dim), dtype=x.dtype, device=x.device)
        if decode_fuses_input(ctx, x.dtype, s.heads, s.kv_heads, s.head_dim, self.runtime.page_size):
            # a pure decode step: the attention kernel norms, rotates and stores q, k, v itself
            paged_attention(qkv, qkv.shape[1], out, cache, group, ctx, s.heads, s.softmax_scale, s.window or 0,
                            raw=(self.q_weight, self.k_weight, self.eps, rot, rotary_dim, slots))
        else:
            ops.qk_norm_rope_cache(qkv, s.heads, s.kv_heads, s.head_dim, self.q_weight, self.k_weight,
                                   self.eps, rot, rotary_dim, slots, cache.k, cache.v, self.runtime.page_size)
            paged_attention(qkv, qkv.shape[1], out, cache, group, ctx, s.heads, s.softmax_scale, s.window or 0)
        if defer_output:
            return ops.linear_or_pending(out, self.wo, self.bo)
        return ops.linear(out, self.wo, bias=self.bo)
