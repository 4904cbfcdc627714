"""The random-weights mode: a model folder (config.json + model.safetensors) from a configuration
and a seed.

Each tensor has a generator of its own, seeded from (seed, tensor name), so a tensor's values do
not depend on which other tensors exist or on their order.  Matrices and tables are N(0, std);
scale vectors of norms are 1, or 1 + N(0, norm_noise).  The reference's test helper fills its tiny
model the same way with its own generator (crates/mrun-engine/src/testing.rs:42-51, 91-149).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Optional, Tuple

import torch

from ..config.spec import ModelSpec, TensorSpec
from .loader import expected_tensors
from .safetensors_io import write_safetensors


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(t: TensorSpec, seed: int, std: float, norm_noise: float, dtype: torch.dtype,
                  device: str = "cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, t.name))
    if t.init == "norm":
        if norm_noise == 0.0:
            return torch.ones(t.shape, dtype=dtype, device=device)
        noise = torch.randn(t.shape, generator=gen, dtype=torch.float32, device=device)
        return (1.0 + norm_noise * noise).to(dtype)
    if t.init != "normal":
        raise ValueError(f"tensor {t.name}: unknown init {t.init!r}")
    if device == "cpu" or len(t.shape) < 2:
        return (torch.randn(t.shape, generator=gen, dtype=torch.float32, device=device) * std).to(dtype)
    # large matrices on the device: row blocks keep the 32-bit staging buffer small
    out = torch.empty(t.shape, dtype=dtype, device=device)
    rows = max(1, (1 << 26) // max(1, out[0].numel()))
    for start in range(0, t.shape[0], rows):
        block = out[start:start + rows]
        block.copy_(torch.randn(block.shape, generator=gen, dtype=torch.float32, device=device) * std)
    return out


def random_tensors(spec: ModelSpec, seed: int, std: float = 0.02, norm_noise: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16, device: str = "cpu"
                   ) -> Iterator[Tuple[str, torch.Tensor]]:
    for t in expected_tensors(spec):
        if t.optional:
            continue
        yield t.name, random_tensor(t, seed, std, norm_noise, dtype, device)


def write_random_model(config, out_dir: str, seed: int, std: float = 0.02, norm_noise: float = 0.0,
                       dtype: str = "bfloat16") -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors`` for a typed configuration."""
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(dtype)
    if torch_dtype is None:
        raise ValueError(f"random weights are written as bfloat16 or float32, got {dtype!r}")
    os.makedirs(out_dir, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      random_tensors(config.to_spec(), seed, std, norm_noise, torch_dtype),
                      metadata={"format": "pt", "seed": str(seed), "std": repr(std),
                                "norm_noise": repr(norm_noise)})
    return out_dir
