"""The attention kernels alone: the CUDA-core kernel (32-bit and bfloat16), the tensor-core prefill
kernel and the split-key decode kernel, against plain softmax attention over gathered keys, with
shuffled pages, odd group sizes, head sizes in steps of 16, windows, and inputs made so that one
far key carries the whole result."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Case:
    """Segments of (context before the step, new tokens) over a shuffled page pool."""

    def __init__(self, segments, heads, kv_heads, head_dim, page_size, dtype, seed=0, window=0, pad=0):
        from mrun_b200.engine.batch import GroupView, HostStaging, SegmentInfo, StepContext
        g = torch.Generator().manual_seed(seed)
        self.heads, self.kv_heads, self.head_dim, self.page_size, self.window = heads, kv_heads, head_dim, page_size, window
        self.dtype = dtype
        total_blocks = sum(-(-(c + n) // page_size) for c, n in segments)
        pages = total_blocks + 5
        order = torch.randperm(pages, generator=g).tolist()
        max_blocks = max(-(-(c + n) // page_size) for c, n in segments) + 2
        slots = len(segments) + 2
        table = torch.full((slots, max_blocks), -1, dtype=torch.int32)
        self.k = (torch.randn(pages, kv_heads, page_size, head_dim, generator=g)).to(dtype)
        self.v = (torch.randn(pages, kv_heads, page_size, head_dim, generator=g)).to(dtype)
        tokens = sum(n for _, n in segments)
        self.q = torch.randn(tokens + pad, heads * head_dim + 24, generator=g).to(dtype)   # a view into a wider buffer
        positions, token_slot, infos = [], [], []
        row = 0
        slot_order = torch.randperm(slots, generator=g).tolist()
        self.seg_pages = []
        for s, (context, new) in enumerate(segments):
            slot = slot_order[s]
            n_blocks = -(-(context + new) // page_size)
            mine = [order.pop() for _ in range(n_blocks)]
            table[slot, :n_blocks] = torch.tensor(mine, dtype=torch.int32)
            self.seg_pages.append(mine)
            positions += list(range(context, context + new))
            token_slot += [slot] * new
            infos.append(SegmentInfo(slot, row, new, context))
            row += new
        positions += [-1] * pad
        token_slot += [0] * pad
        self.segments, self.infos, self.tokens, self.pad = segments, infos, tokens, pad
        self.staging = HostStaging(torch.device(DEV))
        dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        self.table = table.to(DEV)
        self.ctx = StepContext(
            num_tokens=tokens + pad, num_segments=len(segments), segments=infos, token_ids=dev([0] * (tokens + pad)),
            positions=dev(positions), token_slot=dev(token_slot), seg_q_start=dev([0]), seg_kv_len=dev([0]),
            seg_slot=dev([0]), groups={}, max_q_len=max(n for _, n in segments),
            max_kv_len=max(c + n for c, n in segments), page_size=page_size, real_tokens=tokens,
            upload=self.staging.upload)
        self.group = GroupView(self.table, dev([0]), max_blocks)
        self.kd, self.vd, self.qd = self.k.to(DEV), self.v.to(DEV), self.q.to(DEV)

    def keys_of(self, s, cache):
        context, new = self.segments[s]
        rows = [cache[self.seg_pages[s][p // self.page_size], :, p % self.page_size] for p in range(context + new)]
        return torch.stack(rows).float()                       # [S, kv_heads, D]

    def reference(self, scale):
        out = torch.zeros(self.tokens + self.pad, self.heads, self.head_dim)
        group = self.heads // self.kv_heads
        for s, info in enumerate(self.infos):
            k, v = self.keys_of(s, self.k), self.keys_of(s, self.v)
            q = self.q[info.q_start:info.q_start + info.q_len, :self.heads * self.head_dim].float().view(info.q_len, self.heads, self.head_dim)
            for i in range(info.q_len):
                p = info.pos_start + i
                lo = max(0, p - self.window + 1) if self.window else 0
                for h in range(self.heads):
                    scores = (k[lo:p + 1, h // group] @ q[i, h]) * scale
                    out[info.q_start + i, h] = torch.softmax(scores, 0) @ v[lo:p + 1, h // group]
        return out.view(self.tokens + self.pad, -1)

    class Cache:
        pass

    def run(self, scale, force_generic=False):
        from mrun_b200.kernels import ops
        from mrun_b200.kernels.attention import paged_attention
        out = torch.full((self.tokens + self.pad, self.heads * self.head_dim), 3.0, dtype=self.dtype, device=DEV)
        cache = Case.Cache()
        cache.k, cache.v = self.kd, self.vd
        if force_generic:
            ops.paged_attention_generic(self.qd, self.qd.stride(0), out, self.kd, self.vd, self.table,
                                        self.ctx.token_slot, self.ctx.positions, self.heads, scale, self.window)
        else:
            paged_attention(self.qd, self.qd.stride(0), out, cache, self.group, self.ctx, self.heads, scale, self.window)
        return out.float().cpu()


SHAPES = [  # heads, kv_heads, head_dim, page_size
    (4, 2, 16, 16), (6, 3, 32, 8), (7, 1, 48, 4), (8, 8, 64, 32), (10, 2, 80, 16), (32, 8, 128, 16), (2, 1, 256, 16),
    (3, 1, 96, 1), (40, 2, 64, 16), (16, 1, 128, 4), (12, 4, 64, 128), (6, 2, 128, 1), (8, 2, 128, 24)]


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", SHAPES)
@pytest.mark.parametrize("window", [0, 37])
def test_mixed_batch_against_plain(heads, kv_heads, head_dim, page_size, window):
    """Prompt portions beside single tokens, contexts up to a few hundred keys."""
    segments = [(0, 70), (129, 1), (63, 2), (300, 1), (15, 33), (0, 1)]
    scale = head_dim ** -0.5
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        case = Case(segments, heads, kv_heads, head_dim, page_size, dtype, seed=head_dim + window, window=window)
        want = case.reference(scale)
        assert (case.run(scale, force_generic=True) - want).abs().max() <= tol * want.abs().max()
        if dtype == torch.bfloat16:
            assert (case.run(scale) - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", SHAPES)
@pytest.mark.parametrize("window", [0, 100])
def test_decode_batch_against_plain(heads, kv_heads, head_dim, page_size, window):
    """Every segment one token (the split-key kernel where the group fits), with padding rows."""
    segments = [(0, 1), (63, 1), (64, 1), (700, 1), (15, 1), (1023, 1), (200, 1)]
    scale = head_dim ** -0.5
    case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=7 + head_dim, window=window, pad=3)
    want = case.reference(scale)
    got = case.run(scale)
    assert (got[:case.tokens] - want[:case.tokens]).abs().max() <= 2e-2 * want.abs().max()
    assert got[case.tokens:].abs().max() == 0, "padding rows must come out as zeros"
    # the same step again: the plan is made anew and the counters are back at zero
    case.ctx.shared.clear()
    assert (case.run(scale)[:case.tokens] - want[:case.tokens]).abs().max() <= 2e-2 * want.abs().max()


@pytest.mark.parametrize("blocks,min_tiles,splits", [(1, 1, 0), (3, 1, 0), (16, 1, 0), (64, 1, 0), (444, 1, 0), (5, 2, 0),
                                                     (16, 4, 0), (1000, 3, 0), (7, 40, 0),
                                                     (16, 1, 1), (48, 1, 3), (256, 2, 16), (512, 4, 32),
                                                     (26, 1, 32), (40, 1, 2), (64, 3, 32)])
@pytest.mark.parametrize("entry", ["mrun_attn_decode", "mrun_attn_decode_tma"])
def test_decode_tiles_dealt_to_any_number_of_blocks(blocks, min_tiles, splits, entry):
    """The decode kernels (tiles copied by cp.async, tiles brought by TMA into a ring) called directly with forced launch shapes (one block takes every pair,
    several blocks share pairs, more blocks than tiles; tiles dealt across pairs, or every block
    with one pair and the blocks dealt to the pairs by their length), twice in a row (the counters the blocks meet at must be
    back at zero), against the CUDA-core kernel."""
    import ctypes
    from mrun_b200.kernels import lib as L, ops
    from mrun_b200.kernels.ops import _c_float, _c_int, _c_long, _ptr, _stream
    heads, kv_heads, head_dim, page_size = 8, 2, 64, 16
    segments = [(0, 1), (63, 1), (64, 1), (700, 1), (1023, 1), (129, 1)]
    case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=21, pad=2)
    scale = head_dim ** -0.5
    want = case.run(scale, force_generic=True)
    n = case.tokens + case.pad
    library = L.attention(head_dim)
    plan = torch.full((2 * (n + 1) + 1,), -7, dtype=torch.int32, device=DEV)
    assignment = torch.empty(blocks * 8, dtype=torch.int32, device=DEV)
    library.call("mrun_attn_decode_plan", _ptr(case.ctx.positions), _c_int(n), _c_int(0), _c_int(kv_heads),
                 _c_int(blocks), _c_int(min_tiles), _c_int(splits), _ptr(plan), _ptr(assignment), _stream())
    tiles = [1, 1, 2, 11, 16, 3, 0, 0]
    assert plan[:n + 1].tolist() == [0, 1, 2, 4, 15, 31, 34, 34, 34]
    starts = assignment.view(blocks, 2, 4)[:, 0].tolist()
    if splits == 0:
        per = max(-(-68 // blocks), min_tiles)
        assert [s[0] for s in starts] == [min(68, b * per) for b in range(blocks)]    # 34 tiles x 2 kv heads
        assert plan[n + 1:].tolist() == [-7] * (n + 2), "the flat plan writes tokens + 1 numbers"
    else:
        # the fewest tiles a block, at least min_tiles, with which a kv head's pairs fit its blocks
        per_head = blocks // kv_heads
        per = next(p for p in range(max(min_tiles, -(-16 // splits)), 17)
                   if p == 16 or sum(-(-t // p) for t in tiles) <= per_head)
        assert int(plan[2 * (n + 1)]) == per
        pieces = [-(-t // per) for t in tiles]
        assert plan[n + 1:2 * (n + 1)].tolist() == [sum(pieces[:i]) for i in range(n + 1)]
        assert max(s[1] - s[0] for s in starts) <= per
        for b, s in enumerate(starts):                # a block's tiles lie in its own pair
            if s[1] > s[0]:
                first = s[2] * 34 + sum(tiles[:s[3]])
                assert first <= s[0] and s[1] <= first + tiles[s[3]] and s[2] == b // per_head
    assert sum(s[1] - s[0] for s in starts) == 68                                      # every tile dealt once
    part_o = torch.full((blocks, 2, 16, head_dim), float("nan"), device=DEV)
    part_ml = torch.full((blocks, 2, 16, 2), float("nan"), device=DEV)
    counters = torch.zeros(n * kv_heads, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    extra = (_ptr(None), _c_long(case.kd.shape[0]), _ptr(status)) if entry.endswith("tma") else ()
    for _ in range(2):
        out = torch.full((n, heads * head_dim), 3.0, dtype=torch.bfloat16, device=DEV)
        library.call(
            entry, _ptr(case.qd), _c_long(case.qd.stride(0)), _ptr(out), _ptr(case.kd), _ptr(case.vd),
            _ptr(case.table), _c_int(case.group.max_blocks), _ptr(case.ctx.token_slot), _ptr(case.ctx.positions),
            _ptr(plan), _ptr(assignment), _c_int(n), _ptr(part_o), _ptr(part_ml), _ptr(counters), _c_int(blocks),
            _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page_size), _c_float(scale), _c_int(0),
            _c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None), *extra, _stream())
        got = out.float().cpu()
        assert int(status.item()) == 0
        assert (got - want).abs().max() <= 2e-2 * want.abs().max()
        assert got[case.tokens:].abs().max() == 0
        assert int(counters.abs().sum()) == 0


UNEQUAL = [5000, 100, 3000, 64, 9000, 17]       # 79, 2, 47, 2, 141 and 1 tiles of 64 keys


@pytest.mark.parametrize("contexts,blocks,min_tiles,splits,flat", [
    ([0, 63, 64, 700, 1023, 129], 5, 1, 0, True), ([0, 63, 64, 700, 1023, 129], 64, 1, 0, True),
    ([0, 63, 64, 700, 1023, 129], 48, 1, 3, False), ([0, 63, 64, 700, 1023, 129], 26, 1, 32, False),
    (UNEQUAL, 7, 4, 0, True), (UNEQUAL, 296, 4, 0, True),
    (UNEQUAL, 64, 4, 32, False), (UNEQUAL, 16, 4, 32, False), (UNEQUAL, 592, 4, 32, False),
    (UNEQUAL, 16, 1, 2, False)])
@pytest.mark.parametrize("raw", [False, True])
@pytest.mark.parametrize("entry", ["mrun_attn_decode", "mrun_attn_decode_tma"])
def test_decode_contexts_of_unequal_length_and_raw_input(contexts, blocks, min_tiles, splits, flat, raw, entry):
    """The decode kernels called directly over contexts of equal and of very unequal length with
    forced launch shapes; with ``raw`` they take the projection's q, k and v rows and norm, rotate
    and store them themselves, compared with the stand-alone kernel doing that first."""
    from mrun_b200.kernels import lib as L, ops
    from mrun_b200.kernels.ops import _c_float, _c_int, _c_long, _ptr, _stream
    heads, kv_heads, head_dim, page_size, eps, rotary = 8, 2, 64, 16, 1e-5, 48
    case = Case([(c, 1) for c in contexts], heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=5, pad=2)
    scale = head_dim ** -0.5
    n = case.tokens + case.pad
    g = torch.Generator().manual_seed(17)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(n, width, generator=g).to(torch.bfloat16).to(DEV)
    q_weight = (1 + 0.2 * torch.randn(head_dim, generator=g)).to(DEV)
    k_weight = (1 + 0.2 * torch.randn(head_dim, generator=g)).to(DEV)
    angle = torch.rand(n, rotary // 2, generator=g) * 6.28
    rot = torch.stack([angle.cos(), angle.sin()], dim=-1).contiguous().to(DEV)
    slots = [case.seg_pages[s][c // page_size] * page_size + c % page_size for s, c in enumerate(contexts)] + [-1] * case.pad
    slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    library = L.attention(head_dim)

    # what is wanted: the stand-alone kernel norms, rotates and stores, the CUDA-core kernel attends
    k_want, v_want = case.kd.clone(), case.vd.clone()
    if raw:
        q_want = qkv.clone()
        ops.qk_norm_rope_cache(q_want, heads, kv_heads, head_dim, q_weight, k_weight, eps, rot, rotary, slots,
                               k_want, v_want, page_size)
    else:
        q_want = case.qd
    want = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_generic(q_want, q_want.stride(0), want, k_want, v_want, case.table, case.ctx.token_slot,
                                case.ctx.positions, heads, scale, 0)
    want = want.float().cpu()

    plan = torch.empty(2 * (n + 1) + 1, dtype=torch.int32, device=DEV)
    assignment = torch.empty(blocks * 8, dtype=torch.int32, device=DEV)
    library.call("mrun_attn_decode_plan", _ptr(case.ctx.positions), _c_int(n), _c_int(0), _c_int(kv_heads),
                 _c_int(blocks), _c_int(min_tiles), _c_int(splits), _ptr(plan), _ptr(assignment), _stream())
    shape = assignment.view(blocks, 2, 4)[:, 1].tolist()
    assert all((row[2] == 0) == flat for row in shape)
    tiles = sum(c // 64 + 1 for c in contexts) * kv_heads
    assert sum(row[1] - row[0] for row in assignment.view(blocks, 2, 4)[:, 0].tolist()) == tiles
    part_o = torch.full((blocks, 2, 16, head_dim), float("nan"), device=DEV)
    part_ml = torch.full((blocks, 2, 16, 2), float("nan"), device=DEV)
    counters = torch.zeros(n * kv_heads, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    extra = (_ptr(None), _c_long(case.kd.shape[0]), _ptr(status)) if entry.endswith("tma") else ()
    for _ in range(2):
        k_got, v_got = case.kd.clone(), case.vd.clone()
        q_in = qkv if raw else case.qd
        out = torch.full((n, heads * head_dim), 3.0, dtype=torch.bfloat16, device=DEV)
        fused = ((_c_int(1), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(rot), _c_int(rotary), _ptr(slots)) if raw
                 else (_c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None)))
        library.call(
            entry, _ptr(q_in), _c_long(q_in.stride(0)), _ptr(out), _ptr(k_got), _ptr(v_got),
            _ptr(case.table), _c_int(case.group.max_blocks), _ptr(case.ctx.token_slot), _ptr(case.ctx.positions),
            _ptr(plan), _ptr(assignment), _c_int(n), _ptr(part_o), _ptr(part_ml), _ptr(counters), _c_int(blocks),
            _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page_size), _c_float(scale), _c_int(0),
            *fused, *extra, _stream())
        got = out.float().cpu()
        assert int(status.item()) == 0
        assert (got - want).abs().max() <= 2e-2 * want.abs().max()
        assert got[case.tokens:].abs().max() == 0
        assert int(counters.abs().sum()) == 0
        assert (k_got.float() - k_want.float()).abs().max() <= 2e-2 * k_want.float().abs().max()
        assert torch.equal(v_got, v_want)


@pytest.mark.parametrize("cluster", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [(8, 2, 64, 16), (32, 8, 128, 16), (8, 1, 128, 4), (6, 2, 128, 1),
                                                               (12, 4, 64, 128), (3, 3, 64, 32)])
@pytest.mark.parametrize("raw,window", [(False, 0), (True, 0), (False, 100), (True, 200)])
def test_cluster_decode_with_every_cluster_size(cluster, heads, kv_heads, head_dim, page_size, raw, window):
    """The decode kernel that gives every (token, kv head) pair a thread-block cluster, called
    directly with clusters of 1 to 16 blocks over contexts from one key to thousands (pairs with
    fewer tiles than blocks leave blocks without work), with padding rows, windows, and the raw
    q, k, v rows that it norms, rotates and stores itself; twice in a row, against the stand-alone
    kernel followed by the CUDA-core attention.  Twice the same call gives the same bits."""
    from mrun_b200.kernels import lib as L, ops
    from mrun_b200.kernels.ops import _c_float, _c_int, _c_long, _ptr, _stream
    contexts = [0, 63, 64, 700, 1023, 129, 5000, 17]
    eps, rotary = 1e-5, head_dim
    case = Case([(c, 1) for c in contexts], heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=5 + cluster,
                window=window, pad=2)
    scale = head_dim ** -0.5
    n = case.tokens + case.pad
    g = torch.Generator().manual_seed(17)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(n, width, generator=g).to(torch.bfloat16).to(DEV)
    q_weight = (1 + 0.2 * torch.randn(head_dim, generator=g)).to(DEV)
    k_weight = (1 + 0.2 * torch.randn(head_dim, generator=g)).to(DEV)
    angle = torch.rand(n, rotary // 2, generator=g) * 6.28
    rot = torch.stack([angle.cos(), angle.sin()], dim=-1).contiguous().to(DEV)
    slots = [case.seg_pages[s][c // page_size] * page_size + c % page_size for s, c in enumerate(contexts)] + [-1] * case.pad
    slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    library = L.attention(head_dim)
    k_want, v_want = case.kd.clone(), case.vd.clone()
    if raw:
        q_want = qkv.clone()
        ops.qk_norm_rope_cache(q_want, heads, kv_heads, head_dim, q_weight, k_weight, eps, rot, rotary, slots,
                               k_want, v_want, page_size)
    else:
        q_want = case.qd
    want = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_generic(q_want, q_want.stride(0), want, k_want, v_want, case.table, case.ctx.token_slot,
                                case.ctx.positions, heads, scale, window)
    want = want.float().cpu()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = []
    for _ in range(2):
        k_got, v_got = case.kd.clone(), case.vd.clone()
        q_in = qkv if raw else case.qd
        out = torch.full((n, heads * head_dim), 3.0, dtype=torch.bfloat16, device=DEV)
        fused = ((_c_int(1), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(rot), _c_int(rotary), _ptr(slots)) if raw
                 else (_c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None)))
        library.call(
            "mrun_attn_decode_cluster", _ptr(q_in), _c_long(q_in.stride(0)), _ptr(out), _ptr(k_got), _ptr(v_got),
            _ptr(case.table), _c_int(case.group.max_blocks), _ptr(case.ctx.token_slot), _ptr(case.ctx.positions),
            _c_int(n), _c_int(cluster), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page_size),
            _c_float(scale), _c_int(window), *fused, _ptr(None), _c_long(case.kd.shape[0]), _ptr(status), _stream())
        got = out.float().cpu()
        assert int(status.item()) == 0
        assert (got - want).abs().max() <= 2e-2 * want.abs().max()
        assert got[case.tokens:].abs().max() == 0, "padding rows must come out as zeros"
        assert (k_got.float() - k_want.float()).abs().max() <= 2e-2 * k_want.float().abs().max()
        assert torch.equal(v_got, v_want)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])


def test_cluster_decode_refuses_what_it_cannot_take():
    from mrun_b200.kernels import lib as L
    from mrun_b200.kernels.lib import KernelError
    from mrun_b200.kernels.ops import _c_float, _c_int, _c_long, _ptr, _stream
    case = Case([(10, 1)], 32, 2, 64, 16, torch.bfloat16)                       # 16 query heads a kv head
    out = torch.zeros((1, 32 * 64), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    def call(cluster, heads):
        L.attention(64).call(
            "mrun_attn_decode_cluster", _ptr(case.qd), _c_long(case.qd.stride(0)), _ptr(out), _ptr(case.kd), _ptr(case.vd),
            _ptr(case.table), _c_int(case.group.max_blocks), _ptr(case.ctx.token_slot), _ptr(case.ctx.positions),
            _c_int(1), _c_int(cluster), _c_int(heads), _c_int(2), _c_int(64), _c_int(16), _c_float(0.125), _c_int(0),
            _c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None), _ptr(None),
            _c_long(case.kd.shape[0]), _ptr(status), _stream())
    with pytest.raises(KernelError, match="query heads per kv head exceed"):
        call(4, 32)
    with pytest.raises(KernelError, match="cluster of 3 blocks"):
        call(3, 8)


def test_the_router_gives_small_decode_steps_to_clusters_and_large_ones_to_the_plan(monkeypatch):
    """Seven tokens x 8 kv heads fill less than half the device: a cluster a pair, no plan.  With
    the cluster kernel switched off, and for steps with more pairs, the planned kernel runs."""
    from mrun_b200.kernels import attention
    heads, kv_heads, head_dim, page_size = 32, 8, 128, 16
    scale = head_dim ** -0.5
    segments = [(0, 1), (63, 1), (64, 1), (700, 1), (15, 1), (1023, 1), (200, 1)]
    case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=3, pad=1)
    want = case.reference(scale)
    library = attention._lib.attention(head_dim)
    pick = lambda group, tokens, reach=1024: attention.decode_cluster(library, head_dim, group, page_size, tokens, kv_heads, reach)
    assert pick(4, 8) == 4 and pick(4, 1) == 16 and pick(4, 16) == 2
    assert pick(4, 2) == 8                        # sixteen would crowd
    assert pick(4, 19) == 0                       # 152 pairs: more than half the device
    assert pick(16, 1) == 0                       # a group of 16
    # long contexts go to the planned kernel, which cuts a pair into more pieces
    assert pick(4, 8, 4096) == 4 and pick(4, 8, 16384) == 0
    assert pick(4, 1, 4096) == 16 and pick(4, 1, 16384) == 0
    assert pick(4, 4, 16384) == 8 and pick(4, 4, 32768) == 0
    got = case.run(scale)
    assert not any(isinstance(key, tuple) and key[0] == "decode_plan" for key in case.ctx.shared)
    assert (got[:case.tokens] - want[:case.tokens]).abs().max() <= 2e-2 * want.abs().max()
    monkeypatch.setattr(attention, "CLUSTER_DECODE", False)
    case.ctx.shared.clear()
    planned = case.run(scale)
    assert any(isinstance(key, tuple) and key[0] == "decode_plan" for key in case.ctx.shared)
    assert (planned[:case.tokens] - want[:case.tokens]).abs().max() <= 2e-2 * want.abs().max()
    ops_status = attention.ops.tc5_check
    ops_status()


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 65, 127, 255, 256, 400, 511])
def test_one_far_key_among_hundreds_carries_the_result(far):
    """The query is aligned with one key (score far above the rest) whose value is a marker: the
    output must be that marker, for keys at page and tile edges, in every kernel."""
    heads, kv_heads, head_dim, page_size, context = 8, 2, 64, 16, 511
    scale = head_dim ** -0.5
    for segments, label in (([(context, 1)], "decode"), ([(context - 40, 41)], "prefill")):
        for dtype in (torch.float32, torch.bfloat16):
            case = Case(segments, heads, kv_heads, head_dim, page_size, dtype, seed=far)
            page, off = case.seg_pages[0][far // page_size], far % page_size
            direction = torch.randn(head_dim, generator=torch.Generator().manual_seed(1))
            direction /= direction.norm()
            case.k[page, :, off] = (direction * 40.0).to(dtype)
            case.v[page, :, off] = 9.0
            case.q[:, :heads * head_dim] = (direction * 8.0).repeat(heads).to(dtype)
            case.kd, case.vd, case.qd = case.k.to(DEV), case.v.to(DEV), case.q.to(DEV)
            for generic in ((True,) if dtype == torch.float32 else (True, False)):
                got = case.run(scale, force_generic=generic)
                last = got[case.tokens - 1]
                assert (last - 9.0).abs().max() < 0.1, (label, dtype, generic, float(last.min()), float(last.max()))


def test_window_edge():
    """With a window of W the key at p - W + 1 counts and the key at p - W does not."""
    heads, kv_heads, head_dim, page_size, window = 4, 2, 32, 8, 48
    scale = head_dim ** -0.5
    for new in (1, 9):
        for dtype in (torch.float32, torch.bfloat16):
            for inside in (True, False):
                context = 130
                case = Case([(context, new)], heads, kv_heads, head_dim, page_size, dtype, seed=3, window=window)
                p = context + new - 1
                marked = p - window + 1 if inside else p - window
                page, off = case.seg_pages[0][marked // page_size], marked % page_size
                direction = torch.ones(head_dim) / head_dim ** 0.5
                case.k[page, :, off] = (direction * 40.0).to(dtype)
                case.v[page, :, off] = 9.0
                case.q[-1, :heads * head_dim] = (direction * 8.0).repeat(heads).to(dtype)
                case.kd, case.vd, case.qd = case.k.to(DEV), case.v.to(DEV), case.q.to(DEV)
                for generic in ((True,) if dtype == torch.float32 else (True, False)):
                    last = case.run(scale, force_generic=generic)[case.tokens - 1]
                    if inside:
                        assert (last - 9.0).abs().max() < 0.1
                    else:
                        assert last.abs().max() < 5.0, "a key outside the window leaked in"


def test_given_back_pages_are_not_read():
    """Block-table entries of -1 below the window (pages given back) are never dereferenced."""
    heads, kv_heads, head_dim, page_size, window = 4, 1, 64, 16, 40
    scale = head_dim ** -0.5
    for segments in ([(500, 1)], [(480, 21)]):
        case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=11, window=window)
        want = case.reference(scale)
        first_needed = (segments[0][0] - window + 1) // page_size
        slot = case.infos[0].slot
        case.table[slot, :first_needed] = -1
        for generic in (True, False):
            got = case.run(scale, force_generic=generic)
            assert (got - want).abs().max() <= 2e-2 * want.abs().max()
