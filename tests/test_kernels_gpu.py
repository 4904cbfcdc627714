"""Each CUDA kernel alone against a plain 32-bit torch formula of the same operation, at sizes
other than the engine's: widths and vocabularies that are no power of two, head sizes in steps of
16, odd group sizes, several page sizes, windows."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from mrun_b200.kernels import ops as o
    return o


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,hidden", [(37, 24), (509, 100), (1000, 4096)])
def test_embed(dtype, vocab, hidden):
    table = rnd(vocab, hidden, dtype=dtype, seed=1)
    ids = torch.tensor([0, vocab - 1, 5, 5, vocab // 2], dtype=torch.int32, device=DEV)
    out = torch.empty((5, hidden), dtype=torch.float32, device=DEV)
    ops().embed(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden,eps", [(1, 16, 1e-6), (7, 100, 1e-5), (33, 2560, 1e-6), (3, 13000, 1e-3)])
def test_add_rmsnorm(dtype, rows, hidden, eps):
    resid = rnd(rows, hidden, seed=2)
    delta = rnd(rows, hidden, dtype=dtype, seed=3)
    weight = 1 + 0.1 * rnd(hidden, seed=4)
    want_resid = resid + delta.float()
    want = plain.rms_norm(want_resid.cpu(), weight.cpu(), eps).to(DEV)
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    got_resid = resid.clone()
    ops().add_rmsnorm(got_resid, delta, weight, eps, out)
    assert torch.equal(got_resid, want_resid)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert (out.float() - want).abs().max() <= tol * want.abs().max()
    # no delta: the stream stays; chosen rows only: the stream stays too
    keep = resid.clone()
    ops().add_rmsnorm(keep, None, weight, eps, out)
    assert torch.equal(keep, resid)
    index = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    picked = torch.empty((2, hidden), dtype=dtype, device=DEV)
    ops().add_rmsnorm(keep, delta, weight, eps, picked, rows=index)
    assert torch.equal(keep, resid)
    assert (picked.float() - want[[rows - 1, 0]]).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("theta,half", [(10000.0, 8), (1e6, 64), (500000.0, 24)])
def test_rotary_table(theta, half):
    positions = torch.tensor([0, 1, 2, 777, 8191, 40000, -1], dtype=torch.int32, device=DEV)
    inv = (torch.tensor(theta, dtype=torch.float64) ** (-torch.arange(half, dtype=torch.float64) / half)).to(DEV)
    out = torch.empty((7, half, 2), dtype=torch.float32, device=DEV)
    ops().rotary_table(positions, inv, out)
    angle = positions[:6].double()[:, None] * inv[None, :]
    assert (out[:6, :, 0] - angle.cos().float()).abs().max() <= 1.2e-7
    assert (out[:6, :, 1] - angle.sin().float()).abs().max() <= 1.2e-7
    assert torch.equal(out[6, :, 0], torch.ones(half, device=DEV)) and out[6, :, 1].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary_dim,page_size", [
    (4, 2, 16, 16, 16), (6, 3, 32, 32, 8), (5, 5, 48, 24, 4), (8, 1, 128, 128, 16), (3, 1, 80, 80, 32),
    (12, 4, 64, 64, 16), (5, 2, 256, 256, 8), (33, 3, 128, 128, 16), (7, 7, 128, 64, 16)])
def test_qk_norm_rope_cache(dtype, heads, kv_heads, head_dim, rotary_dim, page_size):
    tokens, pages, eps, theta = 11, 9, 1e-5, 10000.0
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rnd(tokens, width, dtype=dtype, seed=5)
    qw, kw = 1 + 0.2 * rnd(head_dim, seed=6), 1 + 0.2 * rnd(head_dim, seed=7)
    positions = torch.tensor([0, 1, 2, 3, 100, 101, 7, 8, 9, 4000, 31], dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * page_size, generator=torch.Generator().manual_seed(8))[:tokens].int().to(DEV)
    slots[3] = -1                                   # a token whose k/v must not be written
    inv = (torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(rotary_dim // 2, dtype=torch.float64) / rotary_dim)).to(DEV)
    rot = torch.empty((tokens, rotary_dim // 2, 2), dtype=torch.float32, device=DEV)
    ops().rotary_table(positions, inv, rot)
    k_cache = torch.full((pages, kv_heads, page_size, head_dim), 7.0, dtype=dtype, device=DEV)
    v_cache = torch.full((pages, kv_heads, page_size, head_dim), 7.0, dtype=dtype, device=DEV)
    src = qkv.float().cpu()
    got = qkv.clone()
    ops().qk_norm_rope_cache(got, heads, kv_heads, head_dim, qw, kw, eps, rot, rotary_dim, slots, k_cache,
                             v_cache, page_size)
    q = src[:, :heads * head_dim].view(tokens, heads, head_dim)
    k = src[:, heads * head_dim:(heads + kv_heads) * head_dim].view(tokens, kv_heads, head_dim)
    v = src[:, (heads + kv_heads) * head_dim:].view(tokens, kv_heads, head_dim)
    pos = positions.cpu()
    want_q = plain.rope(plain.rms_norm(q, qw.cpu(), eps), pos, theta, rotary_dim)
    want_k = plain.rope(plain.rms_norm(k, kw.cpu(), eps), pos, theta, rotary_dim)
    tol = 3e-6 if dtype == torch.float32 else 1.6e-2
    got_q = got[:, :heads * head_dim].float().cpu().view(tokens, heads, head_dim)
    assert (got_q - want_q).abs().max() <= tol * want_q.abs().max()
    # k and v parts of the buffer are left alone
    assert torch.equal(got[:, heads * head_dim:], qkv[:, heads * head_dim:])
    kc, vc = k_cache.float().cpu(), v_cache.float().cpu()
    written = torch.zeros(pages, page_size, dtype=torch.bool)
    for t in range(tokens):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = divmod(s, page_size)
        written[page, off] = True
        assert (kc[page, :, off] - want_k[t]).abs().max() <= tol * want_k.abs().max()
        assert torch.equal(vc[page, :, off], v[t].to(dtype).float())
    assert (kc.permute(0, 2, 1, 3)[~written] == 7.0).all() and (vc.permute(0, 2, 1, 3)[~written] == 7.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,inter", [(1, 8), (5, 200), (17, 9728)])
def test_swiglu(dtype, tokens, inter):
    gate_up = rnd(tokens, 2 * inter, dtype=dtype, seed=9, scale=2.0)
    out = torch.empty((tokens, inter), dtype=dtype, device=DEV)
    ops().swiglu(gate_up, out)
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    want = g * torch.sigmoid(g) * u
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert (out.float() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (3, 509, 96), (65, 130, 257), (128, 64, 64), (200, 1000, 333)])
def test_gemm_f32(m, n, k):
    x, w = rnd(m, k, seed=10), rnd(n, k, seed=11)
    got = ops().gemm_f32_nt(x, w)
    want = (x.double() @ w.double().T)
    assert (got.double() - want).abs().max() <= 1e-6 * want.abs().max() * math.sqrt(k)
    # a row's result does not depend on the other rows in the call
    alone = ops().gemm_f32_nt(x[m // 2:m // 2 + 1].contiguous(), w)
    assert torch.equal(alone[0], got[m // 2])
    # strided input (a view into a wider buffer)
    wide = rnd(m, k + 13, seed=12)
    assert torch.equal(ops().gemm_f32_nt(wide[:, :k], w), ops().gemm_f32_nt(wide[:, :k].contiguous(), w))


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(16, 32), (509, 96), (6144, 4096), (1000, 12288), (24, 160)])
def test_gemm_skinny(m, n, k):
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=20), rnd(n, k, dtype=torch.bfloat16, seed=21, scale=0.05)
    want = x.float() @ w.float().T
    for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 8e-3)):
        got = ops().gemm_skinny(x, w, out_dtype=out_dtype)
        assert got.dtype == out_dtype and got.shape == (m, n)
        assert (got.float() - want).abs().max() <= tol * want.abs().max() * (4 if out_dtype == torch.float32 else 1)
    # a row's result does not depend on the other rows, and a strided x is taken as it is
    alone = ops().gemm_skinny(x[m // 2:m // 2 + 1], w, out_dtype=torch.float32)
    assert torch.equal(alone[0], ops().gemm_skinny(x, w, out_dtype=torch.float32)[m // 2])
    wide = rnd(m, k + 40, dtype=torch.bfloat16, seed=22)
    assert torch.equal(ops().gemm_skinny(wide[:, :k], w), ops().gemm_skinny(wide[:, :k].contiguous(), w))


@pytest.mark.parametrize("m", [1, 8, 13])
@pytest.mark.parametrize("n,k", [(509, 96), (2560, 4096), (4096, 1024), (24, 160)])
def test_gemm_skinny_with_tiles_cut_short(m, n, k):
    """A block of the decode GEMM may take 8 to 15 rows of W instead of its tile's 16, so that a
    product with few rows fills the device evenly: every count gives the bits of the whole tile
    (a row's sum does not depend on which block holds it), in the plain and in the residual
    epilogue, at widths that no count divides."""
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=20), rnd(n, k, dtype=torch.bfloat16, seed=21, scale=0.05)
    whole = o.gemm_skinny(x, w, out_dtype=torch.float32, rows=16)
    want = x.float() @ w.float().T
    assert (whole - want).abs().max() <= 8e-5 * want.abs().max()
    norm_w = 1 + 0.1 * rnd(n, seed=33)
    stream = rnd(m, n, seed=34)
    fusable = n % 32 == 0
    if fusable:
        first = stream.clone()
        rows_whole = o.linear_into_norm(o.PendingLinear(x, w), first, norm_w, 1e-5, rows=16)
    for rows in (0, 8, 9, 11, 14, 15):
        assert torch.equal(o.gemm_skinny(x, w, out_dtype=torch.float32, rows=rows), whole), rows
        if fusable:
            again = stream.clone()
            cut = o.linear_into_norm(o.PendingLinear(x, w), again, norm_w, 1e-5, rows=rows)
            assert torch.equal(again, first) and torch.equal(cut.xw, rows_whole.xw), rows
            # the totals add the same squares in other groups (each group in 32-bit, then as integers)
            assert ((cut.sums[:m] - rows_whole.sums[:m]).abs().double() <= 2e-6 * rows_whole.sums[:m].double()).all(), rows
    with pytest.raises(o.KernelError, match="rows=7"):
        o.gemm_skinny(x, w, rows=7)


@pytest.mark.parametrize("m,inter,k", [(1, 8, 32), (5, 200, 96), (16, 12288, 4096), (9, 9728, 2560)])
def test_gemm_skinny_gated_epilogue(m, inter, k):
    x = rnd(m, k, dtype=torch.bfloat16, seed=23)
    gate, up = rnd(inter, k, dtype=torch.bfloat16, seed=24, scale=0.05), rnd(inter, k, dtype=torch.bfloat16, seed=25, scale=0.05)
    w = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(2 * inter, k).contiguous()
    g = (x.float() @ gate.float().T).bfloat16().float()
    u = (x.float() @ up.float().T).bfloat16().float()
    want = g * torch.sigmoid(g) * u
    got = ops().gemm_skinny(x, w, swiglu_rows=True)
    assert got.shape == (m, inter)
    assert (got.float() - want).abs().max() <= 1.2e-2 * want.abs().max()
    # the unfused pair (product, then activation on the interleaved layout) agrees
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=DEV)
    ops().swiglu(torch.mm(x, w.t()), act, interleaved=True)
    assert (act.float() - want).abs().max() <= 1.2e-2 * want.abs().max()


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("hidden,k,n_next", [(32, 64, 48), (96, 192, 200), (4096, 4096, 6144), (2560, 4096, 9728),
                                             (5120, 1024, 64), (16384, 96, 32)])
def test_gemm_skinny_with_the_residual_sum_and_the_norm_around_it(m, hidden, k, n_next):
    """Three kernels as a decode step chains them: a product whose epilogue adds its result to
    the 32-bit stream and leaves stream * norm weight with per-block sums of squares; the product
    that reads those rows and applies rsqrt(mean + eps) to its own sums; and the same rows
    finished into plain RMSNorm output.  Against x + a W1^T, rmsnorm, · W2^T in 64-bit.  The
    totals of squares are integers, so twice the same call gives the same bits."""
    o = ops()
    eps = 1e-5
    a = rnd(m, k, dtype=torch.bfloat16, seed=30)
    w1 = rnd(hidden, k, dtype=torch.bfloat16, seed=31, scale=0.05)
    w2 = rnd(n_next, hidden, dtype=torch.bfloat16, seed=32, scale=0.05)
    norm_w = 1 + 0.1 * rnd(hidden, seed=33)
    stream = rnd(m, hidden, seed=34, scale=3.0)                        # far from unit scale on purpose
    want_stream = stream.double() + a.double() @ w1.double().T
    normed = want_stream * torch.rsqrt((want_stream ** 2).mean(-1, keepdim=True) + eps) * norm_w.double()
    want = normed @ w2.double().T

    got_stream = stream.clone()
    rows = o.linear_into_norm(o.PendingLinear(a, w1), got_stream, norm_w, eps)
    assert (got_stream.double() - want_stream).abs().max() <= 2e-5 * want_stream.abs().max()
    sums = rows.sums[:m].double() * o.SUMS_UNIT                       # 64-bit fixed point, units of 2^-30
    assert ((sums - (want_stream ** 2).sum(-1)).abs() <= 1e-4 * sums).all()
    assert int(rows.sums[m:].abs().max()) == 0 if m < 16 else True
    finished = rows.finish()
    assert (finished.double() - normed).abs().max() <= 1.2e-2 * normed.abs().max()       # rounded to bfloat16 twice
    for out_dtype, tol in ((torch.float32, 8e-3), (torch.bfloat16, 1.2e-2)):
        got = o.gemm_skinny(rows, w2, out_dtype=out_dtype)
        assert (got.double() - want).abs().max() <= tol * want.abs().max()
    twice = stream.clone()
    rows2 = o.linear_into_norm(o.PendingLinear(a, w1), twice, norm_w, eps)
    assert torch.equal(rows2.sums, rows.sums) and torch.equal(twice, got_stream) and torch.equal(rows2.xw, rows.xw)
    # a row's result depends neither on the other rows nor on how many there are
    alone_stream = stream[m // 2:m // 2 + 1].clone()
    alone = o.linear_into_norm(o.PendingLinear(a[m // 2:m // 2 + 1], w1), alone_stream, norm_w, eps)
    assert torch.equal(alone_stream[0], got_stream[m // 2])
    assert torch.equal(o.gemm_skinny(alone, w2, out_dtype=torch.float32)[0],
                       o.gemm_skinny(rows, w2, out_dtype=torch.float32)[m // 2])
    # chained: the next product's x may itself carry a pending scale
    w3 = rnd(hidden, hidden, dtype=torch.bfloat16, seed=35, scale=0.05)
    again = got_stream.clone()
    o.linear_into_norm(o.PendingLinear(rows, w3), again, norm_w, eps)
    want_again = want_stream + normed @ w3.double().T
    assert (again.double() - want_again).abs().max() <= 8e-3 * want_again.abs().max()
    # the gated epilogue applies the scale before the activation
    if n_next % 16 == 0:
        inter = n_next // 2
        gate, up = w2[:inter], w2[inter:]
        stacked = torch.stack([gate.reshape(-1, 8, hidden), up.reshape(-1, 8, hidden)], dim=1).reshape(n_next, hidden).contiguous()
        g, u = normed @ gate.double().T, normed @ up.double().T
        want_act = g * torch.sigmoid(g) * u
        got_act = o.gemm_skinny(rows, stacked, swiglu_rows=True)
        assert (got_act.double() - want_act).abs().max() <= 2e-2 * want_act.abs().max()


def test_norm_fusion_is_refused_where_it_does_not_fit(monkeypatch):
    o = ops()
    a, w1 = rnd(20, 64, dtype=torch.bfloat16), rnd(64, 64, dtype=torch.bfloat16)
    assert not o.norm_fusable(o.PendingLinear(a, w1), rnd(20, 64), rnd(64))              # more than 16 rows: the vendor GEMM
    monkeypatch.setattr(o, "TC5_GEMM", True)
    a, w1 = rnd(20, 64, dtype=torch.bfloat16), rnd(64, 64, dtype=torch.bfloat16)
    assert o.norm_fusable(o.PendingLinear(a, w1), rnd(20, 64), rnd(64))                  # 17 to 128 rows: the tcgen05 GEMM
    big = rnd(130, 64, dtype=torch.bfloat16)
    assert not o.norm_fusable(o.PendingLinear(big, w1), rnd(130, 64), rnd(64))           # more rows than that
    a = rnd(4, 64, dtype=torch.bfloat16)
    assert o.norm_fusable(o.PendingLinear(a, w1), rnd(4, 64), rnd(64))
    assert not o.norm_fusable(o.PendingLinear(a, rnd(48, 64, dtype=torch.bfloat16)), rnd(4, 48), rnd(48))   # width % 32
    assert not o.norm_fusable(a, rnd(4, 64), rnd(64))                                     # a plain tensor is no pending product
    assert torch.equal(o.PendingLinear(a, w1).compute(), o.linear(a, w1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,inter", [(1, 8), (5, 200), (3, 1001)])
def test_gate_functions(dtype, tokens, inter):
    """The gate's function is a code of the kernels: SiLU and tanh-GELU, stand-alone and in the
    decode GEMM's epilogue; an unknown name is refused."""
    o = ops()
    gate_up = rnd(tokens, 2 * inter, dtype=dtype, seed=9, scale=2.0)
    g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    want = {"silu": g * torch.sigmoid(g) * u,
            "gelu_tanh": 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u}
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    for name, expected in want.items():
        out = torch.empty((tokens, inter), dtype=dtype, device=DEV)
        o.swiglu(gate_up, out, activation=name)
        assert (out.double() - expected).abs().max() <= tol * expected.abs().max(), name
    with pytest.raises(o.KernelError, match="gate function"):
        o.swiglu(gate_up, torch.empty((tokens, inter), dtype=dtype, device=DEV), activation="relu6")
    if dtype == torch.bfloat16 and inter % 8 == 0:
        k = 96
        x = rnd(tokens, k, dtype=dtype, seed=1)
        wg, wu = rnd(inter, k, dtype=dtype, seed=2, scale=0.1), rnd(inter, k, dtype=dtype, seed=3, scale=0.1)
        stacked = torch.stack([wg.view(-1, 8, k), wu.view(-1, 8, k)], dim=1).reshape(2 * inter, k).contiguous()
        g = (x.float() @ wg.float().T).bfloat16().double()
        u = (x.float() @ wu.float().T).bfloat16().double()
        expected = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u
        got = o.gemm_skinny(x, stacked, swiglu_rows=True, activation="gelu_tanh")
        assert (got.double() - expected).abs().max() <= 1.2e-2 * expected.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_with_a_bias(dtype):
    o = ops()
    for m, n, k in ((3, 40, 64), (40, 509, 96)):
        x, w = rnd(m, k, dtype=dtype, seed=1), rnd(n, k, dtype=dtype, seed=2, scale=0.1)
        bias = rnd(n, seed=3)
        want = x.double() @ w.double().T + bias.double()
        got = o.linear(x, w, bias=bias)
        tol = 2e-6 * math.sqrt(k) if dtype == torch.float32 else 1.2e-2
        assert got.dtype == dtype and (got.double() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("m", [1, 17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k,split", [(128, 64, 1), (509, 192, 3), (6144, 4096, 0), (4096, 12288, 0), (1000, 2560, 7),
                                       (24576, 4096, 0), (130, 128, 2), (4096, 4096, 8), (2000, 1024, 5), (40000, 512, 4)])
def test_gemm_tc5(m, n, k, split):
    """The tcgen05 GEMM against a 32-bit product: every token tile, row counts that do not fill a
    tile, widths that do not fill the last 128-row tile, k split over clusters of one to eight
    blocks (0: the library's choice), tiles in one round and in many (inboxes used again)."""
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=30), rnd(n, k, dtype=torch.bfloat16, seed=31, scale=0.05)
    want = x.float() @ w.float().T
    for out_dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 8e-3)):
        got = ops().gemm_tc5(x, w, out_dtype=out_dtype, split=split)
        ops().tc5_check()
        assert got.dtype == out_dtype and got.shape == (m, n)
        assert (got.float() - want).abs().max() <= tol * want.abs().max()
    # the same call again gives the same bits (partial sums add in rank order)
    again = ops().gemm_tc5(x, w, out_dtype=torch.float32, split=split)
    assert torch.equal(again, ops().gemm_tc5(x, w, out_dtype=torch.float32, split=split))
    wide = rnd(m, k + 72, dtype=torch.bfloat16, seed=32)
    assert torch.equal(ops().gemm_tc5(wide[:, :k], w, split=split), ops().gemm_tc5(wide[:, :k].contiguous(), w, split=split))
    # a row's result does not depend on the rows beside it, nor on the token tile they select
    if m > 1:
        alone = ops().gemm_tc5(x[m // 2:m // 2 + 1], w, out_dtype=torch.float32, split=split)
        assert torch.equal(alone[0], again[m // 2])
    ops().tc5_check()


@pytest.mark.parametrize("m,inter,k,split", [(17, 8, 64, 1), (64, 200, 128, 2), (64, 12288, 4096, 0), (128, 1024, 2560, 3),
                                             (40, 3000, 1024, 6)])
def test_gemm_tc5_gated_epilogue(m, inter, k, split):
    x = rnd(m, k, dtype=torch.bfloat16, seed=33)
    gate, up = rnd(inter, k, dtype=torch.bfloat16, seed=34, scale=0.05), rnd(inter, k, dtype=torch.bfloat16, seed=35, scale=0.05)
    w = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(2 * inter, k).contiguous()
    g = (x.float() @ gate.float().T).bfloat16().float()
    u = (x.float() @ up.float().T).bfloat16().float()
    want = g * torch.sigmoid(g) * u
    got = ops().gemm_tc5(x, w, swiglu_rows=True, split=split)
    ops().tc5_check()
    assert got.shape == (m, inter)
    assert (got.float() - want).abs().max() <= 1.2e-2 * want.abs().max()


@pytest.mark.parametrize("m,width,k,inter", [(17, 64, 64, 64), (33, 192, 320, 96), (64, 4096, 4096, 1536), (100, 1024, 2560, 512),
                                             (128, 2560, 1024, 256)])
def test_gemm_tc5_residual_epilogue_and_normed_rows(m, width, k, inter, monkeypatch):
    """A product with the residual sum and the next norm in its epilogue, and the products that
    read its rows with the norm's scale folded in (plain and gated), at 17 to 128 rows, against
    the same in 64-bit; and the same product's stream twice gives the same bits."""
    o = ops()
    monkeypatch.setattr(o, "TC5_GEMM", True)
    a, w1 = rnd(m, k, dtype=torch.bfloat16, seed=40), rnd(width, k, dtype=torch.bfloat16, seed=41, scale=0.05)
    stream = rnd(m, width, seed=42)
    norm_w = 1 + 0.1 * rnd(width, seed=43)
    eps = 1e-5
    want_stream = stream.double() + a.double() @ w1.double().T
    pending = o.PendingLinear(a, w1)
    got_stream = stream.clone()
    assert o.norm_fusable(pending, got_stream, norm_w)
    rows = o.linear_into_norm(pending, got_stream, norm_w, eps)
    o.tc5_check()
    assert isinstance(rows, o.NormedRows) and rows.sums.numel() >= m
    assert (got_stream.double() - want_stream).abs().max() <= 2e-5 * want_stream.abs().max()
    want_sums = (got_stream.double() ** 2).sum(dim=1)
    got_sums = rows.sums[:m].double() * o.SUMS_UNIT
    assert ((got_sums - want_sums).abs() <= 1e-5 * want_sums).all()
    normed = got_stream.double() * torch.rsqrt((got_stream.double() ** 2).mean(dim=1, keepdim=True) + eps) * norm_w.double()
    finished = rows.finish()
    assert (finished.double() - normed).abs().max() <= 1.2e-2 * normed.abs().max()
    w2 = rnd(inter, width, dtype=torch.bfloat16, seed=44, scale=0.05)
    want = normed @ w2.double().T
    got = o.linear(rows, w2, out_dtype=torch.float32)
    assert (got.double() - want).abs().max() <= 1.2e-2 * want.abs().max()
    if inter % 8 == 0:
        up = rnd(inter, width, dtype=torch.bfloat16, seed=45, scale=0.05)
        stacked = torch.stack([w2.view(-1, 8, width), up.view(-1, 8, width)], dim=1).reshape(2 * inter, width).contiguous()
        g, u = normed @ w2.double().T, normed @ up.double().T
        want_act = g * torch.sigmoid(g) * u
        got_act = o.gemm_tc5(rows, stacked, swiglu_rows=True)
        assert (got_act.double() - want_act).abs().max() <= 2e-2 * want_act.abs().max()
    again, first_sums = stream.clone(), rows.sums[:m].clone()
    o.RowSums.begin_step(torch.device(DEV))                  # clears the step's totals, the first call's among them
    rows_again = o.linear_into_norm(pending, again, norm_w, eps)
    assert torch.equal(again, got_stream) and torch.equal(rows_again.xw, rows.xw)
    assert torch.equal(rows_again.sums[:m], first_sums)
    o.tc5_check()


@pytest.mark.parametrize("vocab", [37, 300, 151936])
def test_apply_token_mask(vocab):
    """Rows under a mask keep the logits of their allowed tokens and get -inf elsewhere, tokens
    beyond a narrower mask's vocabulary included; the other rows are untouched."""
    from mrun_b200.sampling import TokenMask
    o = ops()
    logits = rnd(5, vocab, seed=3)
    before = logits.clone()
    g = torch.Generator().manual_seed(vocab)
    masks = [TokenMask.of(torch.randint(0, vocab, (max(1, vocab // 3),), generator=g).tolist(), vocab),
             TokenMask.of([0, vocab // 2, vocab - 5], vocab - 4)]           # a narrower mask: its last token is outside
    rows = [3, 1]
    words_a_mask = -(-vocab // 32)
    words = np.zeros((2, words_a_mask), dtype=np.uint32)
    for m, mask in enumerate(masks):
        words[m, :len(mask.words)] = mask.words
    o.apply_token_mask(logits, torch.tensor(rows, dtype=torch.int32, device=DEV),
                       torch.from_numpy(words.view(np.int32)).to(DEV),
                       torch.tensor([m.vocab for m in masks], dtype=torch.int32, device=DEV))
    got, want = logits.cpu(), before.cpu()
    for row in (0, 2, 4):
        assert torch.equal(got[row], want[row])
    for row, mask in zip(rows, masks):
        allowed = mask.allowed()
        expected = torch.full((vocab,), float("-inf"))
        expected[allowed] = want[row][allowed]
        assert torch.equal(got[row], expected)
    assert masks[1].allowed() == [0, vocab // 2, vocab - 5] and got[1][vocab - 1] == float("-inf")
    # the sampler on masked rows: greedy is the best allowed token, a draw stays inside the mask
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    o.sample(logits, out)
    assert int(out[3]) == max(masks[0].allowed(), key=lambda i: (float(want[3][i]), -i))
    keys = torch.arange(5, dtype=torch.int64, device=DEV) * 977 + 5
    o.sample(logits, out, temperature=torch.full((5,), 1.5, device=DEV), top_p=torch.full((5,), 0.9, device=DEV),
             top_k=torch.full((5,), 7, dtype=torch.int32, device=DEV), min_p=torch.full((5,), 0.01, device=DEV), keys=keys)
    assert masks[0].is_allowed(int(out[3])) and masks[1].is_allowed(int(out[1]))


def test_linear_bf16_accumulates_in_32_bits():
    x, w = rnd(300, 1024, dtype=torch.bfloat16, seed=13), rnd(77, 1024, dtype=torch.bfloat16, seed=14)
    got = ops().linear(x, w, out_dtype=torch.float32)
    want = x.float() @ w.float().T
    assert got.dtype == torch.float32 and (got - want).abs().max() <= 1e-3 * want.abs().max()
    assert ops().linear(x, w).dtype == torch.bfloat16


# --------------------------------------------------------------------------- sampling

@pytest.mark.parametrize("vocab", [7, 509, 151936])
def test_sample_greedy_is_argmax_lowest_index(vocab):
    logits = rnd(5, vocab, seed=15)
    logits[2, 3] = logits[2, vocab - 1] = 50.0                       # a tie: the lower index wins
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops().sample(logits, out)
    want = [int(np.argmax(row)) for row in logits.cpu().numpy()]
    assert out.tolist() == want and want[2] == 3


@pytest.mark.parametrize("vocab", [64, 509, 50000])
def test_sample_temperature_equals_plain_draw(vocab):
    rows = 6
    logits = rnd(rows, vocab, seed=16, scale=2.0)
    temps = [0.8, 1.0, 0.3, 0.0, 1.7, 0.8]
    keys = [plain.draw_key(99, n + 1) for n in range(rows)]
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample(logits, out, temperature=torch.tensor(temps, device=DEV),
                 keys=torch.from_numpy(np.array(keys, dtype=np.uint64).view(np.int64)).to(DEV))
    host = logits.cpu().numpy()
    assert out.tolist() == [plain.sample_token(host[i], temps[i], keys[i]) for i in range(rows)]


def test_sample_filters_keep_the_plain_sets():
    """top-k, top-p and min-p: over many draws every sampled token lies in the plain keep-set, and
    the whole keep-set is reached when it is small."""
    vocab, draws = 97, 400
    row = rnd(1, vocab, seed=17, scale=2.5)
    host = row.cpu().numpy()[0]
    for kwargs in (dict(top_k=5), dict(top_p=0.6), dict(min_p=0.2), dict(top_p=0.9, top_k=8, min_p=0.05)):
        keep = plain.filter_threshold(host, kwargs.get("top_p", 1.0), kwargs.get("top_k", 0), kwargs.get("min_p", 0.0))
        logits = row.expand(draws, vocab).contiguous()
        keys = np.array([plain.draw_key(5, n + 1) for n in range(draws)], dtype=np.uint64)
        out = torch.empty(draws, dtype=torch.int32, device=DEV)
        full = lambda v, dt: torch.full((draws,), v, dtype=dt, device=DEV)
        ops().sample(logits, out, temperature=full(1.5, torch.float32), top_p=full(kwargs.get("top_p", 1.0), torch.float32),
                     top_k=full(kwargs.get("top_k", 0), torch.int32), min_p=full(kwargs.get("min_p", 0.0), torch.float32),
                     keys=torch.from_numpy(keys.view(np.int64)).to(DEV))
        seen = set(out.tolist())
        allowed = set(np.nonzero(keep)[0].tolist())
        assert seen <= allowed, (kwargs, seen - allowed)
        if len(allowed) <= 8:
            assert seen == allowed, (kwargs, allowed - seen)
        want = [plain.sample_token(host, 1.5, int(keys[n]), **kwargs) for n in range(20)]
        assert out.tolist()[:20] == want


def test_repetition_penalty():
    logits = rnd(3, 50, seed=18)
    before = logits.cpu().numpy().copy()
    recent = torch.tensor([[1, 2, 2, -1], [-1, -1, -1, -1], [49, 0, 49, 7]], dtype=torch.int32, device=DEV)
    penalty = torch.tensor([1.3, 1.3, 1.0], device=DEV)
    ops().repetition_penalty(logits, recent, penalty)
    want = before.copy()
    want[0] = plain.apply_repetition_penalty(before[0], [1, 2, 2], 1.3)
    assert np.allclose(logits.cpu().numpy(), want, rtol=1e-6, atol=0)


def test_kernels_refuse_what_they_cannot_take():
    from mrun_b200.kernels import KernelError
    with pytest.raises(KernelError, match="CUDA"):
        ops().swiglu(torch.zeros(2, 8), torch.zeros(2, 4))
    with pytest.raises(KernelError, match="dtype"):
        ops().swiglu(torch.zeros(2, 8, dtype=torch.float16, device=DEV), torch.zeros(2, 4, dtype=torch.float16, device=DEV))
    with pytest.raises(KernelError, match="hidden"):
        big = torch.zeros(1, 60000, device=DEV)
        ops().add_rmsnorm(big, None, torch.ones(60000, device=DEV), 1e-6, torch.empty_like(big))
    with pytest.raises(KernelError, match="rotary_dim"):
        ops().qk_norm_rope_cache(torch.zeros(1, 48, device=DEV), 1, 1, 16, None, None, 0.0,
                                 torch.zeros(1, 2, 2, device=DEV), 5, None, None, None, 4)


@pytest.mark.parametrize("rows,vocab,n", [(1, 7, 3), (3, 509, 5), (2, 151936, 2), (4, 1000, 1000), (2, 33, 40)])
def test_top_logprobs(rows, vocab, n):
    logits = rnd(rows, vocab, seed=vocab + n) * 3.0
    logits[0, min(5, vocab - 1)] = logits[0, 0]                  # a tie: the smaller id comes first
    ids, values = ops().top_logprobs(logits, n)
    n_eff = min(n, vocab)
    assert ids.shape == (rows, n_eff) and values.shape == (rows, n_eff)
    for row in range(rows):
        want = plain.top_logprobs(logits[row].cpu().numpy(), n)
        assert ids[row].tolist() == [i for i, _ in want]
        assert np.abs(values[row].cpu().numpy() - np.array([v for _, v in want])).max() <= 2e-5
