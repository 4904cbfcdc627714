"""From a model folder to an :class:`Executor`: config.json picks the architecture, the weights
are bound by name (crates/mrun-engine/src/nuvec_engine.rs:282-363 is the reference's load path)."""
from __future__ import annotations

from typing import Optional

from .. import registry
from ..weights import load_tensors, random_tensors
from .executor import Executor


def executor_from_folder(model_dir: str, dtype: str = "bfloat16", page_size: int = 16,
                         num_pages: int = 256, max_requests: int = 8, device: str = "cuda:0",
                         sizing=None) -> Executor:
    config = registry.load_config(model_dir)
    spec = config.to_spec()
    tensors = load_tensors(model_dir, spec)
    executor = Executor(spec, tensors, dtype=dtype, page_size=page_size, num_pages=num_pages,
                        max_requests=max_requests, device=device, sizing=sizing)
    executor.config = config
    return executor


def executor_from_config(config, seed: int, dtype: str = "bfloat16", std: float = 0.02,
                         norm_noise: float = 0.0, page_size: int = 16, num_pages: int = 256,
                         max_requests: int = 8, device: str = "cuda:0", sizing=None) -> Executor:
    """Random weights made on the device, without a folder (large shapes for measurement).  The
    values differ from the folder-writing mode's, which draws on the host."""
    import torch
    spec = config.to_spec()
    store = torch.bfloat16 if dtype in ("bfloat16", "bf16") else torch.float32
    tensors = dict(random_tensors(spec, seed, std, norm_noise, store, device=device))
    executor = Executor(spec, tensors, dtype=dtype, page_size=page_size, num_pages=num_pages,
                        max_requests=max_requests, device=device, sizing=sizing)
    executor.config = config
    return executor
