"""The decode attention entry point that allocates nothing (``mrun_attn_decode_static``).

Some programs that embed this library cannot ask for device memory when they call it: the host
application owns all of the device's memory through an arena of its own, or runs a loop that
cannot afford an allocation's synchronisation, or sits in a server callback that forbids
allocating.  For them the library keeps the scratch of the split-key decode kernel in a fixed
array of its own.  This test calls that entry point through its exported C symbol, twice in a
row (the array keeps the first call's contents), and checks the output against the ordinary entry
point's, which gets its scratch from the caller.  It also checks that a call beyond the array's
stated size is refused with a message rather than run.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def call_decode(dll, name, case, out, blocks, min_tiles, scratch=None):
    """``scratch``: (plan, assignment, part_o, part_ml, counters) for the ordinary entry point, None
    for the one that brings its own."""
    from mrun_b200.kernels.ops import _c_float, _c_int, _c_long, _ptr, _stream
    fn = getattr(dll, name)
    fn.restype = ctypes.c_int
    n = case.tokens + case.pad
    head = (_ptr(case.qd), _c_long(case.qd.stride(0)), _ptr(out), _ptr(case.kd), _ptr(case.vd), _ptr(case.table),
            _c_int(case.group.max_blocks), _ptr(case.ctx.token_slot), _ptr(case.ctx.positions))
    shape = (_c_int(case.heads), _c_int(case.kv_heads), _c_int(case.head_dim), _c_int(case.page_size),
             _c_float(case.head_dim ** -0.5), _c_int(case.window))
    if scratch is None:
        return fn(*head, _c_int(n), _c_int(blocks), _c_int(min_tiles), *shape, _stream())
    plan, assignment, part_o, part_ml, counters = scratch
    # the ordinary entry point also takes the description of raw q, k, v rows; here q is ready
    ready = (_c_int(0), _ptr(None), _ptr(None), _c_float(0.0), _ptr(None), _c_int(0), _ptr(None))
    return fn(*head, _ptr(plan), _ptr(assignment), _c_int(n), _ptr(part_o), _ptr(part_ml), _ptr(counters),
              _c_int(blocks), *shape, *ready, _stream())


@pytest.mark.parametrize("head_dim,blocks,min_tiles,window", [(64, 5, 1, 0), (128, 16, 2, 0), (32, 3, 1, 100), (128, 444, 4, 0)])
def test_static_scratch_entry_point_matches_the_ordinary_one(head_dim, blocks, min_tiles, window):
    from mrun_b200.kernels import lib
    from test_attention_gpu import Case
    heads, kv_heads, page_size = 8, 2, 16
    segments = [(0, 1), (63, 1), (64, 1), (700, 1), (1023, 1), (129, 1), (300, 1)]
    case = Case(segments, heads, kv_heads, head_dim, page_size, torch.bfloat16, seed=31 + head_dim, window=window, pad=2)
    library = lib.attention(head_dim)
    dll = ctypes.CDLL(library.path)                      # the exported C symbols, nothing in between
    last_error = dll.mrun_last_error
    last_error.restype = ctypes.c_char_p
    n = case.tokens + case.pad

    want = torch.full((n, heads * head_dim), 3.0, dtype=torch.bfloat16, device=DEV)
    from mrun_b200.kernels.ops import _c_int, _ptr, _stream
    plan = torch.empty(n + 1, dtype=torch.int32, device=DEV)
    assignment = torch.empty(blocks * 8, dtype=torch.int32, device=DEV)
    library.call("mrun_attn_decode_plan", _ptr(case.ctx.positions), _c_int(n), _c_int(window), _c_int(kv_heads),
                 _c_int(blocks), _c_int(min_tiles), _c_int(0), _ptr(plan), _ptr(assignment), _stream())
    part_o = torch.empty((blocks, 2, 16, head_dim), dtype=torch.float32, device=DEV)
    part_ml = torch.empty((blocks, 2, 16, 2), dtype=torch.float32, device=DEV)
    counters = torch.zeros(n * kv_heads, dtype=torch.int32, device=DEV)
    assert call_decode(dll, "mrun_attn_decode", case, want, blocks, min_tiles,
                       (plan, assignment, part_o, part_ml, counters)) == 0
    torch.cuda.synchronize()
    plain = case.reference(head_dim ** -0.5)
    assert (want.float().cpu() - plain).abs().max() <= 2e-2 * plain.abs().max()

    for attempt in range(2):                             # the second call finds the first call's leftovers
        got = torch.full((n, heads * head_dim), 5.0, dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = call_decode(dll, "mrun_attn_decode_static", case, got, blocks, min_tiles)
        assert rc == 0, last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before       # nothing through torch's allocator
        if attempt == 1:
            # nor through the driver: the device's free memory is what it was (the first call
            # looked the array up and loaded the kernel, which may take memory once)
            assert torch.cuda.mem_get_info()[0] == free_before
        assert (got.float() - want.float()).abs().max().item() <= 2e-2 * plain.abs().max().item(), attempt
        assert torch.equal(got, want), "same kernel, same merge order: the bits should agree"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from mrun_b200.kernels import lib
    from test_attention_gpu import Case
    case = Case([(10, 1)] * 40, 16, 2, 64, 16, torch.bfloat16, seed=3)
    dll = ctypes.CDLL(lib.attention(64).path)
    last_error = dll.mrun_last_error
    last_error.restype = ctypes.c_char_p
    out = torch.zeros((case.tokens, 16 * 64), dtype=torch.bfloat16, device=DEV)
    assert call_decode(dll, "mrun_attn_decode_static", case, out, 513, 1) != 0      # more blocks than it has scratch for
    assert b"exceeds the built-in scratch" in last_error()
    assert float(out.abs().max()) == 0.0                                               # nothing ran
    assert call_decode(dll, "mrun_attn_decode_static", case, out, 512, 1) == 0
