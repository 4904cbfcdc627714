"""Each part a layer is put together from, built alone from its spec and compared with the plain
function of the same part: norm, rotary table, attention, gated feed-forward, block, whole model."""
from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from tiny_models import TINY, tiny_config

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype, page_size=8):
    from mrun_b200.parts import Precision, Runtime
    return Runtime(torch.device(DEV), Precision.of(dtype), page_size)


def one_request_context(mixers, tokens, rt, chunks=None):
    """A cache manager with one entry per mixer and the step context(s) of one request fed whole,
    or in the given chunk sizes."""
    from mrun_b200.cache import CacheManager
    from mrun_b200.engine.batch import HostStaging, StepEntry, build_context
    needs = [m.cache_need() for m in mixers]
    manager = CacheManager(needs, [None] * len(needs), rt.page_size, 64, 2, device=rt.device, dtype=rt.precision.act)
    staging = HostStaging(rt.device)
    request = manager.admit("r")
    for n in (chunks or [len(tokens)]):
        start = request.length
        plan = manager.plan_append([(request, n)])
        ctx = build_context([StepEntry(request, tokens[start:start + n])], manager, staging)
        yield ctx, manager, start, n
        manager.commit(plan)


def tolerance(dtype):
    return 3e-5 if dtype == "float32" else 3e-2


def weights_for(name, seed=1):
    from mrun_b200.weights import random_tensors
    config = tiny_config(name)
    t = TINY[name]
    tensors = dict(random_tensors(config.to_spec(), seed, std=t["std"], norm_noise=0.1, dtype=torch.bfloat16))
    return config, tensors, {k: v.float() for k, v in tensors.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from mrun_b200.config import RMSNormSpec
    from mrun_b200.parts import NORMS
    rt = runtime(dtype)
    weight = 1 + 0.1 * torch.randn(100)
    norm = NORMS.build(RMSNormSpec(100, 1e-5), {"weight": weight}, rt)
    resid = torch.randn(7, 100, device=DEV)
    delta = torch.randn(7, 100, device=DEV).to(rt.precision.act)
    want_resid = resid + delta.float()
    want = plain.rms_norm(want_resid.cpu(), weight, 1e-5)
    got = norm.add_forward(resid, delta)
    assert got.dtype == rt.precision.act and torch.equal(resid, want_resid)
    assert (got.float().cpu() - want).abs().max() <= tolerance(dtype) * want.abs().max()
    rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    picked = norm.rows_forward(resid, None, rows)
    assert (picked.float().cpu() - want[[6, 2]]).abs().max() <= tolerance(dtype) * want.abs().max()
    assert (norm.forward(want_resid.to(rt.precision.act)).float().cpu() - want).abs().max() <= 2 * tolerance(dtype) * want.abs().max()


def test_rotary_part():
    from mrun_b200.config import RotarySpec
    from mrun_b200.parts import POSITIONS
    rt = runtime("float32")
    rotary = POSITIONS.build(RotarySpec(32, 24, 5e5), {}, rt)
    assert rotary.rotary_dim == 24
    for ctx, *_ in one_request_context([], list(range(40)), rt, chunks=[33, 7]):
        table = rotary.rotation(ctx)
        assert rotary.rotation(ctx) is table                      # made once per step, then shared
        pos = ctx.positions.cpu().double()
        inv = torch.tensor(5e5, dtype=torch.float64) ** (-2.0 * torch.arange(12, dtype=torch.float64) / 24)
        angle = pos[:, None] * inv[None, :]
        assert (table[..., 0].cpu() - angle.cos().float()).abs().max() <= 1.2e-7
        assert (table[..., 1].cpu() - angle.sin().float()).abs().max() <= 1.2e-7
    with pytest.raises(ValueError, match="rotary_dim"):
        POSITIONS.build(RotarySpec(32, 33, 1e4), {}, rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
@pytest.mark.parametrize("chunks", [None, [5, 2, 30, 1, 12], [11] + [1] * 39, [1] * 50])
def test_attention_part(dtype, name, chunks):
    from mrun_b200.parts import MIXERS
    from mrun_b200.parts.base import local
    config, tensors, w = weights_for(name)
    rt = runtime(dtype, TINY[name]["page_size"])
    spec = config.to_spec().layers[0].mixer
    prefix = "model.layers.0.self_attn"
    mixer = MIXERS.build(spec, local(tensors, prefix), rt)
    L = 50                                              # every list of chunks adds up to it
    h = torch.randn(L, config.hidden_size).to(torch.bfloat16)
    want = plain.attention_block(h.float(), w, prefix, config.to_dict(), torch.arange(L))
    got = torch.empty(L, config.hidden_size)
    for ctx, manager, start, n in one_request_context([mixer], [0] * L, rt, chunks):
        out = mixer.forward(h[start:start + n].to(DEV).to(rt.precision.act), ctx, manager.entries[0])
        got[start:start + n] = out.float().cpu()
    assert (got - want).abs().max() <= tolerance(dtype) * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
@pytest.mark.parametrize("rows", [3, 40])
def test_gated_mlp_part(dtype, name, rows):
    from mrun_b200.parts import FEED_FORWARDS
    from mrun_b200.parts.base import local
    config, tensors, w = weights_for(name)
    rt = runtime(dtype)
    prefix = "model.layers.1.mlp"
    mlp = FEED_FORWARDS.build(config.to_spec().layers[1].feed_forward, local(tensors, prefix), rt)
    h = torch.randn(rows, config.hidden_size).to(torch.bfloat16)
    want = plain.swiglu_mlp(h.float(), w, prefix)
    got = mlp.forward(h.to(DEV).to(rt.precision.act), None).float().cpu()
    assert (got - want).abs().max() <= tolerance(dtype) * want.abs().max()
    # a gate function that no kernel has is refused when the part is built, by name
    from dataclasses import replace
    from mrun_b200.kernels.lib import KernelError
    with pytest.raises(KernelError, match="gate function 'erf_gelu'.*silu"):
        FEED_FORWARDS.build(replace(config.to_spec().layers[1].feed_forward, activation="erf_gelu"), local(tensors, prefix), rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_block_and_model(dtype, name):
    from mrun_b200.engine.model import Model
    from mrun_b200.parts import ARRANGEMENTS
    config, tensors, w = weights_for(name)
    rt = runtime(dtype, TINY[name]["page_size"])
    spec = config.to_spec()
    L = 37
    # one block: stream in, stream + both branches out
    block = ARRANGEMENTS.get("pre_norm")(spec.layers[1], tensors, rt)
    x = (torch.randn(L, config.hidden_size) * 0.3)
    want = plain.decoder_layer(x, w, 1, config.to_dict(), torch.arange(L))
    for ctx, manager, start, n in one_request_context([block.mixer], [0] * L, rt):
        resid = x.to(DEV).clone()
        delta = block.forward(resid, None, ctx, manager.entries[0])
        if not isinstance(delta, torch.Tensor):            # the last product, left for the next norm to run
            delta = delta.compute()
        got = (resid + delta.float()).cpu()
    assert (got - want).abs().max() <= tolerance(dtype) * want.abs().max()
    # the whole model on one request, cut in two steps
    model = Model(spec, tensors, rt)
    tokens = torch.randint(0, config.vocab_size, (L,), generator=torch.Generator().manual_seed(4)).tolist()
    want = plain.forward(config.to_dict(), w, tokens)
    assert model.graph_safe and len(model.cache_needs()) == config.num_hidden_layers
    mixers = [b.mixer for b in model.blocks]
    got = torch.empty(L, config.vocab_size)
    for ctx, manager, start, n in one_request_context(mixers, tokens, rt, chunks=[20, 17]):
        rows = torch.arange(n, dtype=torch.int32, device=DEV)
        got[start:start + n] = model.forward(ctx, manager.entries, rows).cpu()
    assert (got - want).abs().max() <= tolerance(dtype) * want.abs().max()
