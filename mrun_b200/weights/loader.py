"""Binding checkpoint tensors to a model by name.

The expected set comes from the model's parts (``tensor_specs``).  Everything that does not fit is
reported in one error: tensors that are missing, tensors the model does not use, and tensors of
the wrong shape (the reference fails on the first missing name and on leftovers,
crates/mrun-engine/src/load.rs:202-206, crates/mrun-engine/src/models/common.rs:433-438).

Storage dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16
is widened to 32-bit (exactly; the run's precision decides later whether a matrix is narrowed to
bfloat16, so a float16 checkpoint run in 32-bit computes with the stored values), integer tables
become int32.  A stored output head of a model with tied embeddings is dropped
(crates/mrun-engine/src/models/common.rs:367-369).  Tensors whose names the spec ignores (vision
tower, multi-token-prediction heads, rotary frequency tables) are never read
(crates/mrun-engine/src/load.rs:168-173); a part's optional tensors (a linear layer's ``.bias``)
are bound when the checkpoint has them (crates/mrun-engine/src/load.rs:281).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..config.spec import ModelSpec, TensorSpec
from .safetensors_io import SafetensorsFile, iter_tensors, open_model_files


class WeightsError(ValueError):
    def __init__(self, where: str, architecture: str, missing: List[str], unexpected: List[str],
                 wrong: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"weights in {where} do not match {architecture}:"]
        for title, names in (("missing", missing), ("unexpected", unexpected), ("wrong shape", wrong)):
            if names:
                shown = ", ".join(names[:12]) + (f", ... (+{len(names) - 12} more)" if len(names) > 12 else "")
                lines.append(f"  {title} ({len(names)}): {shown}")
        super().__init__("\n".join(lines))


def expected_tensors(spec: ModelSpec) -> List[TensorSpec]:
    """Every tensor the model binds, in a fixed order (embedding, head, layers, final norm)."""
    from ..parts import ARRANGEMENTS, NORMS, TRANSFORMS
    out = [TensorSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size))]
    if not spec.tie_embeddings:
        out.append(TensorSpec(spec.head_name, (spec.vocab_size, spec.hidden_size)))
    for layer in spec.layers:
        out += ARRANGEMENTS.get(layer.arrangement).tensor_specs(layer)
    out += NORMS.tensor_specs(spec.final_norm, spec.final_norm_prefix)
    for transform in (spec.embedding_transform, spec.logits_transform):
        if transform is not None:
            out += TRANSFORMS.tensor_specs(transform, getattr(transform, "prefix", ""))
    names = [t.name for t in out]
    if len(set(names)) != len(names):
        raise ValueError("two parts of the model bind the same tensor name")
    return out


def _keep_dtype(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.dtype in (torch.bfloat16, torch.float32):
        return tensor
    if tensor.dtype == torch.float16:
        return tensor.to(torch.float32)
    if tensor.dtype == torch.float64:
        return tensor.to(torch.float32)
    if tensor.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.int32):
        return tensor.to(torch.int32)
    raise ValueError(f"dtype {tensor.dtype} is not a weight dtype")


def bind(spec: ModelSpec, available: Dict[str, object], where: str, fetch) -> Dict[str, torch.Tensor]:
    """``available``: name -> shape of what the checkpoint holds; ``fetch(name)`` reads one."""
    expected = expected_tensors(spec)
    names = {t.name for t in expected}
    dropped_head = {spec.head_name} if spec.tie_embeddings else set()
    head_stem = spec.head_name.rsplit(".", 1)[0] + "."
    missing, wrong = [], []
    for t in expected:
        if t.name not in available:
            if not t.optional:
                missing.append(t.name)
        elif tuple(available[t.name]) != tuple(t.shape):
            wrong.append(f"{t.name}: file {list(available[t.name])}, expected {list(t.shape)}")
    unexpected = sorted(
        n for n in available
        if n not in names and not spec.ignores(n)
        and not (spec.tie_embeddings and (n in dropped_head or n.startswith(head_stem))))
    if missing or unexpected or wrong:
        raise WeightsError(where, spec.architecture, missing, unexpected, wrong)
    return {t.name: _keep_dtype(fetch(t.name)) for t in expected if t.name in available}


def load_tensors(model_dir: str, spec: ModelSpec) -> Dict[str, torch.Tensor]:
    files = open_model_files(model_dir)
    owner: Dict[str, SafetensorsFile] = {}
    for name, f in iter_tensors(files):
        owner[name] = f            # a later file wins, as a merged map would
    shapes = {name: f.info(name)[1] for name, f in owner.items()}
    return bind(spec, shapes, model_dir, lambda name: owner[name].tensor(name))


def bind_tensors(spec: ModelSpec, tensors: Dict[str, torch.Tensor], where: str = "memory") -> Dict[str, torch.Tensor]:
    """The same checks for tensors that are already in memory."""
    return bind(spec, {n: tuple(t.shape) for n, t in tensors.items()}, where, lambda name: tensors[name])
