"""Interfaces of the parts a layer is put together from, and the registries that map a spec's
``kind`` to the class that builds it.

A part is built from ``(spec, tensors, runtime)``: its spec carries every size and constant, the
tensors are the checkpoint's under the part's own local names, the runtime says where and in which
precision to compute.  No part knows which model it is in.

Roles and what each must provide
--------------------------------
every part      ``tensor_specs(spec, prefix) -> list[TensorSpec]`` (static): the checkpoint tensors
                it binds, with full names.
norm            ``forward(x) -> y``; ``add_forward(resid, delta) -> y`` adds ``delta`` (may be
                None) into the 32-bit residual stream in place and returns the normed rows in the
                activation dtype; ``rows_forward(resid, delta, rows) -> y`` does so for the rows
                named by an int32 index tensor without touching the stream.
position        ``rotary_dim`` and ``rotation(ctx) -> float32 [tokens, rotary_dim // 2, 2]``
                (cos, sin) per token and pair (j, j + rotary_dim // 2), computed once per step
                and shared by all layers through ``ctx.shared``.
mixer           ``cache_need() -> PagedKV | FixedState | None`` and
                ``forward(x, ctx, cache) -> y`` with x, y ``[tokens, hidden]`` in the activation
                dtype; ``cache`` is the schedule entry's :class:`EntryCache`
                (``writable`` False when it reads another entry's cache).
                ``graph_safe`` tells whether forward issues the same device work for every step
                of the same shape (no host-side branching on the batch's contents).
feed-forward    ``forward(x, ctx) -> y``.
arrangement     a block class built from a :class:`LayerSpec`; ``forward(resid, delta, ctx,
                cache) -> delta`` takes the stream and the branch output not yet added to it and
                returns the next pending branch output.
transform       ``forward(x) -> x`` on the 32-bit stream right after the embedding
                (``ModelSpec.embedding_transform``: a scale, an added table) or on the float32
                logits of the wanted rows (``ModelSpec.logits_transform``: a soft cap, a bias);
                may work in place.

Optional capabilities (class attributes, all off when absent), which let a step of a handful of
rows fold the residual sum and the norm into the products around them:
``can_defer_output`` on a mixer or feed-forward (``forward(..., defer_output=True)`` may return its
last product unrun, ``kernels.ops.PendingLinear``); ``accepts_pending`` on a norm or arrangement
(``delta`` may be such a product; a norm may answer with ``kernels.ops.NormedRows``);
``accepts_normed_rows`` on a mixer or feed-forward (``x`` may be ``NormedRows``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Optional

import torch


@dataclass(frozen=True)
class Precision:
    name: str                 # "bfloat16" | "float32"
    act: torch.dtype          # activations, matrix weights, key/value pages
    logits: torch.dtype = torch.float32

    @staticmethod
    def of(name: str) -> "Precision":
        if name in ("bfloat16", "bf16"):
            return Precision("bfloat16", torch.bfloat16)
        if name in ("float32", "fp32", "f32"):
            return Precision("float32", torch.float32)
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")


@dataclass
class Runtime:
    device: torch.device
    precision: Precision
    page_size: int

    def matrix(self, tensor: torch.Tensor) -> torch.Tensor:
        """A checkpoint matrix in the compute dtype on the device."""
        return tensor.to(device=self.device, dtype=self.precision.act).contiguous()

    def vector_f32(self, tensor: torch.Tensor) -> torch.Tensor:
        """A scale vector: always 32-bit on the device (norm arithmetic is 32-bit)."""
        return tensor.to(device=self.device, dtype=torch.float32).contiguous()


class Registry:
    def __init__(self, role: str):
        self.role = role
        self._classes: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def add(cls: type) -> type:
            self._classes[kind] = cls
            return cls
        return add

    def get(self, kind: str) -> type:
        try:
            return self._classes[kind]
        except KeyError:
            raise KeyError(f"no {self.role} of kind {kind!r} is registered "
                           f"(known: {', '.join(sorted(self._classes)) or 'none'})") from None

    def build(self, spec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        return self.get(spec.kind)(spec, tensors, runtime)

    def tensor_specs(self, spec, prefix: str):
        return self.get(spec.kind).tensor_specs(spec, prefix)

    def kinds(self):
        return sorted(self._classes)


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
ARRANGEMENTS = Registry("arrangement")
TRANSFORMS = Registry("transform")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_arrangement = ARRANGEMENTS.register
register_transform = TRANSFORMS.register


def local(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    """The tensors under ``prefix.`` with the prefix removed."""
    dot = prefix + "."
    return {name[len(dot):]: t for name, t in tensors.items() if name.startswith(dot)}
