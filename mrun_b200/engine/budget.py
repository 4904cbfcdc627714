"""Memory budget: how much of the GPU the engine takes and how many tokens of cache that leaves.

The rules follow the reference's budget module (crates/mrun-engine/src/budget.rs):

* the automatic budget is the smaller of ``physical − 2 GiB`` and ``available − margin`` with
  ``margin = clamp(physical ÷ 8, 2 GiB, 6 GiB)`` (budget.rs:97-101, 172-189; the "recommended
  working set" term is a Metal figure and has no counterpart on this device);
* ``--budget-gib`` lowers it and cannot raise it (budget.rs:105-109, 191-224);
* ``--context`` lowers it to what that many tokens need beside the weights and the scratch, and
  is refused when that does not fit, naming the largest context that does (budget.rs:321-359);
* the token capacity is what the budget leaves after weights and scratch, divided by the bytes a
  token holds in every cache group, at most the model's maximum position (budget.rs:261-303);
* a model must leave room for ``INITIAL_STATE_TOKENS`` of cache (budget.rs:20-21, 238-259).

Everything here is arithmetic on byte counts; the only device call is :func:`read_device`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

GIB = 1 << 30
SYSTEM_GUARD = 2 * GIB          # always left to the system
INITIAL_STATE_TOKENS = 4096     # the cache a model must leave room for


class BudgetError(ValueError):
    """A budget or context that cannot be honoured; the message names the figures."""


@dataclass(frozen=True)
class DeviceMemory:
    physical: int
    available: Optional[int] = None     # free right now; None when it was not read


@dataclass(frozen=True)
class MemoryBudget:
    budget: int             # bytes the engine may hold in total
    binding: str            # which term set it: "physical", "available", "budget-gib", "context"
    weights: int = 0
    scratch: int = 0
    cache: int = 0          # bytes left for pages
    capacity_tokens: int = 0

    def breakdown(self) -> dict:
        return {"budget_bytes": self.budget, "binding": self.binding, "weights_bytes": self.weights,
                "scratch_bytes": self.scratch, "cache_bytes": self.cache, "capacity_tokens": self.capacity_tokens}


def gib(n: int) -> str:
    """``4.30 GiB``, as the refusals print sizes (budget.rs:167-170)."""
    return f"{n / GIB:.2f} GiB"


def margin(physical: int) -> int:
    return min(max(physical // 8, 2 * GIB), 6 * GIB)


def automatic(device: DeviceMemory) -> tuple[int, str]:
    best, binding = max(0, device.physical - SYSTEM_GUARD), "physical"
    if device.available is not None:
        room = max(0, device.available - margin(device.physical))
        if room < best:
            best, binding = room, "available"
    return best, binding


def plan(device: DeviceMemory, budget_gib: Optional[int] = None) -> MemoryBudget:
    """The top-level budget: :func:`automatic`, lowered by ``budget_gib``."""
    auto, binding = automatic(device)
    if budget_gib is None:
        return MemoryBudget(auto, binding)
    if budget_gib < 1:
        raise BudgetError("--budget-gib must be at least 1")
    wanted = budget_gib * GIB
    if wanted > auto:
        raise BudgetError(f"--budget-gib {budget_gib} is above the automatic budget of {gib(auto)} "
                          f"(set by {binding} memory); it can only lower the budget")
    return MemoryBudget(wanted, "budget-gib")


def scratch_estimate(hidden: int, activation_elements: int, vocab: int, max_batch_tokens: int,
                     max_requests: int, bytes_per_element: int) -> int:
    """Activations of the largest step plus fixed working memory: per token the 32-bit stream,
    its normed copy and a branch output, and the widest temporaries any part declares; the logits
    of every live request twice (one step in flight while the last is read); and 256 MiB for the
    vendor library's workspace, attention partials and staging."""
    per_token = hidden * (4 + 2 * bytes_per_element) + activation_elements * bytes_per_element
    return max_batch_tokens * per_token + 2 * max_requests * vocab * 4 + 256 * (1 << 20)


def with_capacity(budget: MemoryBudget, weights: int, scratch: int, bytes_per_token: int,
                  max_tokens: Optional[int] = None, fixed_state: int = 0) -> MemoryBudget:
    """Completes ``budget`` with what the weights and the scratch leave for the cache.
    ``max_tokens`` caps the capacity (the model's maximum position times the requests it may
    hold); ``fixed_state`` is the per-request state of fixed size, held for every slot."""
    left = budget.budget - weights - scratch - fixed_state
    need = INITIAL_STATE_TOKENS * bytes_per_token
    if max_tokens is not None:
        need = min(need, max_tokens * bytes_per_token)
    if left < need:
        raise BudgetError(f"the model does not fit: weights {gib(weights)} + scratch {gib(scratch)} + "
                          f"{min(INITIAL_STATE_TOKENS, max_tokens or INITIAL_STATE_TOKENS)} tokens of cache "
                          f"{gib(need)} need {gib(weights + scratch + fixed_state + need)}, the budget is "
                          f"{gib(budget.budget)}")
    tokens = left // bytes_per_token if bytes_per_token else 0
    if max_tokens is not None:
        tokens = min(tokens, max_tokens)
    return MemoryBudget(budget.budget, budget.binding, weights, scratch + fixed_state, tokens * bytes_per_token, tokens)


def for_context(budget: MemoryBudget, context: int, weights: int, scratch: int, bytes_per_token: int,
                max_tokens: Optional[int] = None, fixed_state: int = 0) -> MemoryBudget:
    """Lowers ``budget`` to what ``context`` tokens need, so that the capacity is exactly that."""
    if context < 1:
        raise BudgetError("--context must be at least 1 token")
    if max_tokens is not None and context > max_tokens:
        raise BudgetError(f"--context {context} is beyond the {max_tokens} tokens this model can hold")
    need = weights + scratch + fixed_state + context * bytes_per_token
    if need > budget.budget:
        largest = max(0, (budget.budget - weights - scratch - fixed_state) // max(1, bytes_per_token))
        raise BudgetError(f"--context {context} needs {gib(need)} (weights {gib(weights)}, scratch {gib(scratch)}, "
                          f"cache {gib(context * bytes_per_token)}); the budget is {gib(budget.budget)}, "
                          f"the largest context that fits is {largest} tokens")
    return MemoryBudget(need, "context", weights, scratch + fixed_state, context * bytes_per_token, context)


def read_device(device: str = "cuda:0") -> DeviceMemory:
    import torch
    free, total = torch.cuda.mem_get_info(torch.device(device))
    return DeviceMemory(physical=int(total), available=int(free))
