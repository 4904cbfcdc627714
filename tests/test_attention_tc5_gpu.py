"""The tcgen05 prefill attention alone (head sizes 64 and 128): long prompt portions over many
128-key tiles against plain softmax attention, with groups that do and do not divide the 128-row
tile, shuffled pages of odd sizes, windows, several requests in one launch, row maxima that grow
from tile to tile (the lazy rescale of the accumulator), one far key that carries the result, and
agreement with the mma.sync kernel it replaces."""
from __future__ import annotations

import pytest
import torch

from test_attention_gpu import DEV, Case

pytestmark = pytest.mark.gpu


def reference(case: Case, scale: float) -> torch.Tensor:
    """Plain attention per segment, whole matrices at once (the loops of Case.reference take
    minutes at these lengths)."""
    out = torch.zeros(case.tokens + case.pad, case.heads, case.head_dim, dtype=torch.float64)
    group = case.heads // case.kv_heads
    for s, info in enumerate(case.infos):
        k, v = case.keys_of(s, case.k).double(), case.keys_of(s, case.v).double()        # [S, kvh, D]
        q = case.q[info.q_start:info.q_start + info.q_len, :case.heads * case.head_dim].double()
        q = q.view(info.q_len, case.heads, case.head_dim)
        pos = torch.arange(info.pos_start, info.pos_start + info.q_len)
        keys = torch.arange(k.shape[0])
        seen = keys[None, :] <= pos[:, None]
        if case.window:
            seen &= keys[None, :] >= (pos[:, None] - case.window + 1)
        for h in range(case.heads):
            scores = (q[:, h] @ k[:, h // group].T) * scale
            scores = scores.masked_fill(~seen, float("-inf"))
            out[info.q_start:info.q_start + info.q_len, h] = torch.softmax(scores, -1) @ v[:, h // group]
    return out.view(case.tokens + case.pad, -1).float()


def uses_tcgen05(head_dim: int, ratio: int, page_size: int) -> bool:
    from mrun_b200.kernels import lib
    from mrun_b200.kernels.attention import prefill_uses_tcgen05
    return prefill_uses_tcgen05(lib.attention(head_dim), head_dim, ratio, page_size)


def check_status():
    from mrun_b200.kernels import ops
    ops.tc5_check(torch.device(DEV))


SHAPES = [  # heads, kv_heads, head_dim, page_size
    (32, 8, 128, 16), (8, 8, 128, 16), (6, 2, 128, 4), (4, 4, 64, 8), (40, 8, 64, 16), (14, 2, 64, 32),
    (16, 1, 128, 16), (8, 2, 128, 128), (4, 2, 64, 256), (4, 1, 128, 1), (6, 3, 64, 2)]


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", SHAPES)
@pytest.mark.parametrize("window", [0, 200])
def test_long_portions_against_plain(heads, kv_heads, head_dim, page_size, window):
    assert uses_tcgen05(head_dim, heads // kv_heads, page_size)
    segments = [(0, 530), (700, 300), (1, 1), (250, 129), (1000, 40), (130, 2)]
    scale = head_dim ** -0.5
    case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=heads + window, window=window)
    want = reference(case, scale)
    got = case.run(scale)
    check_status()
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()


def test_growing_maxima_rescale_the_accumulator():
    """Keys further along have larger scores, by far more than the rescale step, so the running
    maximum of every row moves at every tile; the outputs must still match."""
    heads, kv_heads, head_dim, page_size = 8, 2, 128, 16
    scale = head_dim ** -0.5
    case = Case([(0, 900)], heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=5)
    direction = torch.ones(head_dim) / head_dim ** 0.5
    for p in range(900):
        page, off = case.seg_pages[0][p // page_size], p % page_size
        case.k[page, :, off] += (direction * (p / 900.0) * 120.0).to(torch.bfloat16)
    case.q[:, :heads * head_dim] += (direction * 6.0).repeat(heads).to(torch.bfloat16)
    case.kd, case.qd = case.k.to(DEV), case.q.to(DEV)
    want = reference(case, scale)
    got = case.run(scale)
    check_status()
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()


@pytest.mark.parametrize("far", [0, 127, 128, 129, 255, 256, 383, 640, 1023])
def test_one_far_key_carries_the_result(far):
    heads, kv_heads, head_dim, page_size, context = 8, 2, 128, 16, 1024
    scale = head_dim ** -0.5
    case = Case([(context - 200, 200)], heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=far)
    page, off = case.seg_pages[0][far // page_size], far % page_size
    direction = torch.randn(head_dim, generator=torch.Generator().manual_seed(1))
    direction /= direction.norm()
    case.k[page, :, off] = (direction * 40.0).to(torch.bfloat16)
    case.v[page, :, off] = 9.0
    case.q[:, :heads * head_dim] = (direction * 8.0).repeat(heads).to(torch.bfloat16)
    case.kd, case.vd, case.qd = case.k.to(DEV), case.v.to(DEV), case.q.to(DEV)
    got = case.run(scale)
    check_status()
    first_seeing = max(0, far - (context - 200))                 # the first new token at or after the key
    rows = got[first_seeing:case.tokens]
    assert (rows - 9.0).abs().max() < 0.1


def test_agrees_with_the_mma_sync_kernel(monkeypatch):
    from mrun_b200.kernels import attention
    heads, kv_heads, head_dim, page_size = 32, 8, 128, 16
    scale = head_dim ** -0.5
    case = Case([(0, 777), (300, 100)], heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=9)
    new = case.run(scale)
    check_status()
    monkeypatch.setattr(attention, "TC5_PREFILL", False)
    case.ctx.shared.clear()
    old = case.run(scale)
    assert (new - old).abs().max() <= 2e-2 * old.abs().max()


def test_other_page_sizes_take_the_older_kernel():
    assert not uses_tcgen05(128, 4, 24)
    case = Case([(0, 300)], 8, 2, 128, 24, torch.bfloat16, seed=2)
    want = reference(case, 128 ** -0.5)
    assert (case.run(128 ** -0.5) - want).abs().max() <= 2e-2 * want.abs().max()


def test_given_back_pages_are_not_read():
    heads, kv_heads, head_dim, page_size, window = 8, 2, 128, 16, 150
    scale = head_dim ** -0.5
    case = Case([(600, 200)], heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=11, window=window)
    want = reference(case, scale)
    first_needed = (600 - window + 1) // page_size
    case.table[case.infos[0].slot, :first_needed] = -1
    got = case.run(scale)
    check_status()
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()


def test_single_tokens_beside_portions_take_the_decode_kernel(monkeypatch):
    """A step of prompt portions and single decode tokens at long contexts: the single tokens go
    through the split-key decode kernel as a selection of the step's rows, the portions through
    the prefill kernels, and every row agrees with plain attention either way."""
    from mrun_b200.kernels import attention
    heads, kv_heads, head_dim, page_size = 32, 8, 128, 16
    scale = head_dim ** -0.5
    segments = [(0, 300), (2000, 1), (513, 1), (64, 1), (100, 40), (4095, 1), (7, 2)]
    case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=13)
    want = reference(case, scale)
    got = case.run(scale)
    check_status()
    rows, positions, slots, n = case.ctx.shared["single_tokens"]
    assert n == 4 and rows.tolist() == [300, 301, 302, 343] and positions.tolist() == [2000, 513, 64, 4095]
    # four single tokens x 8 kv heads: a cluster a pair, no plan
    assert not any(key[0] == "decode_plan" for key in case.ctx.shared if isinstance(key, tuple))
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()
    # the planned decode kernel over the same selection of rows
    monkeypatch.setattr(attention, "CLUSTER_DECODE", False)
    case.ctx.shared.clear()
    planned = case.run(scale)
    check_status()
    assert any(key[0] == "decode_plan" and key[-1] for key in case.ctx.shared if isinstance(key, tuple))
    assert (planned - want).abs().max() <= 2e-2 * want.abs().max()
    # the same step with the decode kernel switched off: the 64-row tiles take the single tokens
    monkeypatch.setattr(attention, "TMA_DECODE", False)
    case.ctx.shared.clear()
    other = case.run(scale)
    assert "single_tokens" not in case.ctx.shared
    assert (other - want).abs().max() <= 2e-2 * want.abs().max()
