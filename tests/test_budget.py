"""The memory budget's arithmetic (no device): the automatic budget and its binding term, the
override that may only lower it, the capacity beside weights and scratch, and the refusals."""
import pytest

from mrun_b200.cache import FixedState, PagedKV, token_bytes
from mrun_b200.engine import budget
from mrun_b200.engine.budget import GIB, BudgetError, DeviceMemory


def test_automatic_budget_and_its_binding_term():
    # 180 GiB device, all of it free: what is free less the 6 GiB margin binds
    device = DeviceMemory(physical=180 * GIB, available=180 * GIB)
    assert budget.margin(device.physical) == 6 * GIB
    assert budget.automatic(device) == (174 * GIB, "available")
    assert budget.automatic(DeviceMemory(180 * GIB)) == (178 * GIB, "physical")
    # another process holds 100 GiB: what is free less the margin binds
    assert budget.automatic(DeviceMemory(180 * GIB, 80 * GIB)) == (74 * GIB, "available")
    # small devices: the margin is an eighth, at least 2 GiB
    assert budget.margin(8 * GIB) == 2 * GIB and budget.margin(32 * GIB) == 4 * GIB
    assert budget.automatic(DeviceMemory(3 * GIB, 1 * GIB)) == (0, "available")


def test_budget_gib_lowers_and_never_raises():
    device = DeviceMemory(80 * GIB, 80 * GIB)
    auto, _ = budget.automatic(device)
    assert budget.plan(device).budget == auto
    lowered = budget.plan(device, 40)
    assert lowered.budget == 40 * GIB and lowered.binding == "budget-gib"
    with pytest.raises(BudgetError, match="above the automatic budget of 74.00 GiB"):
        budget.plan(device, 75)
    with pytest.raises(BudgetError):
        budget.plan(device, 0)


def test_capacity_is_what_weights_and_scratch_leave():
    top = budget.plan(DeviceMemory(80 * GIB), 20)
    per_token = 144 * 1024                      # the 8B shape: 36 layers x 2 x 8 heads x 128 x 2 bytes
    done = budget.with_capacity(top, weights=16 * GIB, scratch=1 * GIB, bytes_per_token=per_token)
    assert done.capacity_tokens == (3 * GIB) // per_token
    assert done.cache == done.capacity_tokens * per_token and done.weights == 16 * GIB
    # capped by what the model can address
    capped = budget.with_capacity(top, 16 * GIB, 1 * GIB, per_token, max_tokens=8192)
    assert capped.capacity_tokens == 8192
    # per-request state of fixed size is held for every slot
    stateful = budget.with_capacity(top, 16 * GIB, 1 * GIB, per_token, fixed_state=1 * GIB)
    assert stateful.capacity_tokens == (2 * GIB) // per_token and stateful.scratch == 2 * GIB
    # a model must leave room for 4096 tokens of cache
    with pytest.raises(BudgetError, match="does not fit"):
        budget.with_capacity(top, 19 * GIB, 1 * GIB - 1, per_token)
    # ... unless it cannot hold that many anyway
    tiny = budget.with_capacity(top, 19 * GIB, GIB - 600 * per_token, per_token, max_tokens=512)
    assert tiny.capacity_tokens == 512


def test_context_sets_the_budget_or_names_the_largest_that_fits():
    top = budget.plan(DeviceMemory(80 * GIB), 20)
    per_token = 144 * 1024
    done = budget.for_context(top, 16384, 16 * GIB, 1 * GIB, per_token, max_tokens=40960)
    assert done.capacity_tokens == 16384 and done.binding == "context"
    assert done.budget == 17 * GIB + 16384 * per_token
    largest = (3 * GIB) // per_token
    with pytest.raises(BudgetError, match=f"largest context that fits is {largest} tokens"):
        budget.for_context(top, 32768, 16 * GIB, 1 * GIB, per_token, max_tokens=40960)
    with pytest.raises(BudgetError, match="beyond the 40960 tokens"):
        budget.for_context(top, 65536, 16 * GIB, 1 * GIB, per_token, max_tokens=40960)
    with pytest.raises(BudgetError):
        budget.for_context(top, 0, 16 * GIB, 1 * GIB, per_token)


def test_token_bytes_counts_owning_entries_only():
    needs = [PagedKV(8, 128), PagedKV(8, 128, window=64), None, FixedState((4, 16)), PagedKV(2, 64)]
    shares = [None, None, 0, None, None]
    per_token, per_slot = token_bytes(needs, shares, 2)
    assert per_token == 2 * 8 * 128 * 2 * 2 + 2 * 2 * 64 * 2
    assert per_slot == 4 * 16 * 4
    # the reference's figure for the 8B shape: 144 KiB a token (registry.rs:305)
    assert token_bytes([PagedKV(8, 128)] * 36, [None] * 36, 2)[0] == 144 * 1024


def test_scratch_estimate_grows_with_the_step_and_the_vocabulary():
    small = budget.scratch_estimate(4096, 3 * 12288, 151936, 2048, 8, 2)
    assert budget.scratch_estimate(4096, 3 * 12288, 151936, 4096, 8, 2) > small
    assert budget.scratch_estimate(4096, 3 * 12288, 151936, 2048, 64, 2) - small == 2 * 56 * 151936 * 4
    assert small > 256 * (1 << 20)
