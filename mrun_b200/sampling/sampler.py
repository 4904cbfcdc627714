"""Chooses one token per logits row on the device with the sampling kernels."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import REPETITION_CONTEXT, SamplingParams, draw_key


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draws: Sequence[int], recent: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``logits``: float32 [rows, vocab] (penalties are applied in place).  ``seeds[i]`` and
        ``draws[i]`` (counted from 1) key row i's draw.  ``recent[i]``: the request's last token
        ids for the repetition penalty.  Returns int32 [rows] on the device."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.greedy and p.repetition_penalty == 1.0 for p in params):
            return ops.sample(logits, out)
        keys = np.zeros(rows, dtype=np.uint64)
        for i, p in enumerate(params):
            keys[i] = draw_key(seeds[i], draws[i]) if not p.greedy else 0
        f32 = lambda values: torch.tensor(values, dtype=torch.float32).to(self.device, non_blocking=True)
        if any(p.repetition_penalty != 1.0 for p in params):
            table = np.full((rows, REPETITION_CONTEXT), -1, dtype=np.int32)
            for i, ids in enumerate(recent or []):
                ids = list(ids)[-REPETITION_CONTEXT:]
                table[i, :len(ids)] = ids
            ops.repetition_penalty(logits, torch.from_numpy(table).to(self.device),
                                   f32([p.repetition_penalty for p in params]))
        return ops.sample(
            logits, out,
            temperature=f32([p.temperature for p in params]),
            top_p=f32([p.top_p for p in params]),
            top_k=torch.tensor([p.top_k for p in params], dtype=torch.int32).to(self.device),
            min_p=f32([p.min_p for p in params]),
            keys=torch.from_numpy(keys.view(np.int64)).to(self.device))

    def top_logprobs(self, logits: torch.Tensor, n: int):
        """(ids int32 [rows, n], log-probabilities float32 [rows, n]) of each row's n most likely
        tokens, most likely first, ties by the smaller id; on the device."""
        return ops.top_logprobs(logits, n)
