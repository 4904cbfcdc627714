"""Parts and arrangements that are not Qwen3's, defined here and run without a change to the
framework: a mixer that keeps state of a fixed size per request (registered from this file), a
rotary encoding with its own table, attention with a window, a layer that runs twice, a layer
that reads the cache another run wrote, and a feed-forward that routes each token to two of five
experts.  The toy model is compared with a plain whole-sequence
implementation under several ways of cutting the work."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB, EPS, THETA, WINDOW = 48, 4, 2, 16, 80, 101, 1e-5, 1e4, 9


# ------------------------------------------------------------------ toy parts (test-side only)

@dataclass(frozen=True)
class DecaySpec:
    """state_t = decay * state_{t-1} + W x_t ; y_t = state_t : one vector of state per request."""
    kind: ClassVar[str] = "toy_decay"
    hidden: int
    decay: float


@dataclass(frozen=True)
class HalfStepRotarySpec:
    """Rotary positions that advance half a step per token."""
    kind: ClassVar[str] = "toy_half_step_rotary"
    head_dim: int
    rotary_dim: int
    theta: float


def register_toy_parts():
    from mrun_b200.cache import FixedState
    from mrun_b200.config import TensorSpec
    from mrun_b200.parts import register_mixer, register_position

    @register_mixer("toy_decay")
    class DecayMixer:
        graph_safe = False                     # walks the step's segments on the host

        @staticmethod
        def tensor_specs(spec, prefix):
            return [TensorSpec(f"{prefix}.in_proj.weight", (spec.hidden, spec.hidden))]

        def __init__(self, spec, tensors, runtime):
            self.spec = spec
            self.weight = tensors["in_proj.weight"].to(runtime.device, torch.float32)

        def cache_need(self):
            return FixedState((self.spec.hidden,), "float32")

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            projected = x.float() @ self.weight.T
            for seg in ctx.segments:
                state = cache.state[seg.slot]
                for row in range(seg.q_start, seg.q_start + seg.q_len):
                    state.mul_(self.spec.decay).add_(projected[row])
                    out[row] = state.to(x.dtype)
            return out

    @register_position("toy_half_step_rotary")
    class HalfStepRotary:
        @staticmethod
        def tensor_specs(spec, prefix):
            return []

        def __init__(self, spec, tensors, runtime):
            self.spec, self.rotary_dim = spec, spec.rotary_dim
            half = spec.rotary_dim // 2
            self.inv = (torch.tensor(spec.theta, dtype=torch.float64)
                        ** (-2.0 * torch.arange(half, dtype=torch.float64) / spec.rotary_dim)).to(runtime.device)

        def rotation(self, ctx):
            key = ("toy_half_step_rotary", self.spec)
            if key not in ctx.shared:
                angle = ctx.positions.double()[:, None] * 0.5 * self.inv[None, :]
                ctx.shared[key] = torch.stack([angle.cos(), angle.sin()], dim=-1).float().contiguous()
            return ctx.shared[key]


def toy_spec():
    from mrun_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec,
                                  ScheduleEntry)
    norm, mlp = RMSNormSpec(HIDDEN, EPS), GatedMLPSpec(HIDDEN, INTER)
    full = AttentionSpec(HIDDEN, HEADS, KV_HEADS, HEAD_DIM, HEAD_DIM ** -0.5, RMSNormSpec(HEAD_DIM, EPS),
                         RotarySpec(HEAD_DIM, HEAD_DIM, THETA), None)
    windowed = AttentionSpec(HIDDEN, HEADS, KV_HEADS, HEAD_DIM, HEAD_DIM ** -0.5, None,
                             HalfStepRotarySpec(HEAD_DIM, 8, THETA), WINDOW)
    layers = (
        LayerSpec("model.layers.0", full, mlp, norm, norm),
        LayerSpec("model.layers.1", DecaySpec(HIDDEN, 0.9), mlp, norm, norm, mixer_prefix="decay"),
        LayerSpec("model.layers.2", windowed, mlp, norm, norm),
    )
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1), ScheduleEntry(0, cache_of=0))
    return ModelSpec("ToyForCausalLM", VOCAB, HIDDEN, 512, layers, norm, tie_embeddings=False, schedule=schedule)


# ------------------------------------------------------------------ the plain toy model

def plain_attention(h, w, prefix, positions, qk_norm, rotary_dim, step, window, shared_kv=None):
    L = h.shape[0]
    q = (h @ w[f"{prefix}.q_proj.weight"].T).view(L, HEADS, HEAD_DIM)
    k = (h @ w[f"{prefix}.k_proj.weight"].T).view(L, KV_HEADS, HEAD_DIM)
    v = (h @ w[f"{prefix}.v_proj.weight"].T).view(L, KV_HEADS, HEAD_DIM)
    if qk_norm:
        q = plain.rms_norm(q, w[f"{prefix}.q_norm.weight"], EPS)
        k = plain.rms_norm(k, w[f"{prefix}.k_norm.weight"], EPS)
    scaled = positions.double() * step
    q, k = plain.rope(q, scaled, THETA, rotary_dim), plain.rope(k, scaled, THETA, rotary_dim)
    if shared_kv is not None:
        k, v = shared_kv
    o = plain.attention_scores_softmax_values(q, k, v, HEAD_DIM ** -0.5, positions, window)
    return o.reshape(L, HEADS * HEAD_DIM) @ w[f"{prefix}.o_proj.weight"].T, (k, v)


def plain_toy(w, tokens):
    positions = torch.arange(len(tokens))
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    norm = lambda x, name: plain.rms_norm(x, w[name], EPS)

    def feed_forward(x, i):
        return x + plain.swiglu_mlp(norm(x, f"model.layers.{i}.post_attention_layernorm.weight"), w, f"model.layers.{i}.mlp")

    def decay(x):
        h = norm(x, "model.layers.1.input_layernorm.weight") @ w["model.layers.1.decay.in_proj.weight"].T
        state, rows = torch.zeros(HIDDEN), []
        for row in h:
            state = 0.9 * state + row
            rows.append(state)
        return feed_forward(x + torch.stack(rows), 1)

    a, kv0 = plain_attention(norm(x, "model.layers.0.input_layernorm.weight"), w, "model.layers.0.self_attn",
                             positions, True, HEAD_DIM, 1.0, None)
    x = feed_forward(x + a, 0)
    x = decay(x)
    a, _ = plain_attention(norm(x, "model.layers.2.input_layernorm.weight"), w, "model.layers.2.self_attn",
                           positions, False, 8, 0.5, WINDOW)
    x = feed_forward(x + a, 2)
    x = decay(x)                                                   # the second run has state of its own
    a, _ = plain_attention(norm(x, "model.layers.0.input_layernorm.weight"), w, "model.layers.0.self_attn",
                           positions, True, HEAD_DIM, 1.0, None, shared_kv=kv0)
    x = feed_forward(x + a, 0)
    return norm(x, "model.norm.weight") @ w["lm_head.weight"].T


# ------------------------------------------------------------------ the test

@pytest.mark.parametrize("dtype,tolerance", [("float32", 3e-5), ("bfloat16", 4e-2)])
def test_toy_model_with_parts_of_its_own(dtype, tolerance):
    from mrun_b200.cache import FixedState, PagedKV
    from mrun_b200.engine import Executor, StepEntry
    from mrun_b200.weights import expected_tensors, random_tensors
    register_toy_parts()
    spec = toy_spec()
    names = {t.name for t in expected_tensors(spec)}
    assert "model.layers.1.decay.in_proj.weight" in names and "model.layers.2.self_attn.q_norm.weight" not in names
    tensors = dict(random_tensors(spec, seed=3, std=0.08, norm_noise=0.1))
    w = {k: v.float() for k, v in tensors.items()}
    ex = Executor(spec, tensors, dtype=dtype, page_size=4, num_pages=80, max_requests=3)
    assert not ex.model.graph_safe and not ex.use_graphs

    needs = ex.model.cache_needs()
    assert [type(n) for n in needs] == [PagedKV, FixedState, PagedKV, FixedState, type(None)]
    assert set(ex.cache.groups) == {("paged", None), ("paged", WINDOW)}
    assert ex.cache.entries[4].k is ex.cache.entries[0].k and not ex.cache.entries[4].writable
    assert ex.cache.entries[1].state is not ex.cache.entries[3].state

    gen = torch.Generator().manual_seed(9)
    seqs = {name: torch.randint(0, VOCAB, (n,), generator=gen).tolist() for name, n in (("a", 61), ("b", 37), ("c", 50))}
    want = {name: plain_toy(w, tokens) for name, tokens in seqs.items()}
    scale = max(float(x.abs().max()) for x in want.values())

    def check(name, start, logits):
        got = logits.cpu()
        error = float((got - want[name][start:start + got.shape[0]]).abs().max()) / scale
        assert error <= tolerance, (name, start, error)

    # whole
    r = ex.admit("whole")
    check("a", 0, ex.step([StepEntry(r, seqs["a"], range(61))]))
    ex.release(r)
    # portions of changing size, then token by token; the window gives pages back on the way
    r = ex.admit("portions")
    at = 0
    for n in (2, 7, 3, 16, 5, 2, 9) + (1,) * 17:
        check("a", at, ex.step([StepEntry(r, seqs["a"][at:at + n], range(n))]))
        at += n
    assert at == 61
    held = len(r.pages_held(("paged", WINDOW)))
    assert held <= -(-WINDOW // 4) + 1 and len(r.pages_held(("paged", None))) == 16
    ex.release(r)
    # mixed: three live requests, portions of some beside single tokens of others, slots reused
    live = {name: ex.admit(name) for name in seqs}
    fed = {name: 0 for name in seqs}
    sizes = {"a": [30, 1, 1, 13, 1, 1, 14], "b": [1, 1, 20, 1, 14], "c": [5, 40, 1, 1, 1, 1, 1]}
    for turn in range(7):
        entries, names = [], []
        for name in seqs:
            if turn < len(sizes[name]):
                n = sizes[name][turn]
                entries.append(StepEntry(live[name], seqs[name][fed[name]:fed[name] + n], range(n)))
                names.append((name, fed[name], n))
                fed[name] += n
        logits = ex.step(entries)
        row = 0
        for name, start, n in names:
            check(name, start, logits[row:row + n])
            row += n
    assert fed == {name: len(tokens) for name, tokens in seqs.items()}
    for request in live.values():
        ex.release(request)
    ex.cache.check_invariants()
    assert ex.cache.free_pages(("paged", None)) == 80 and ex.cache.free_pages(("paged", WINDOW)) == 80
    # a new request in a used slot starts from zero state
    r = ex.admit("again")
    check("b", 0, ex.step([StepEntry(r, seqs["b"], range(37))]))
    ex.release(r)


# ------------------------------------------------------------------ a feed-forward with routing

EXPERTS, TOP = 5, 2


@dataclass(frozen=True)
class RoutedSpec:
    """y = sum over the token's TOP experts of gate_e * down_e(silu(gate_proj_e x) * up_proj_e x);
    gates = softmax of the router's logits over the chosen experts, in 32-bit."""
    kind: ClassVar[str] = "toy_routed"
    hidden: int
    intermediate: int
    experts: int
    top: int


def register_routed():
    from mrun_b200.config import TensorSpec
    from mrun_b200.parts import register_feed_forward

    @register_feed_forward("toy_routed")
    class RoutedFeedForward:
        @staticmethod
        def tensor_specs(spec, prefix):
            specs = [TensorSpec(f"{prefix}.router.weight", (spec.experts, spec.hidden))]
            for e in range(spec.experts):
                specs += [TensorSpec(f"{prefix}.experts.{e}.gate_proj.weight", (spec.intermediate, spec.hidden)),
                          TensorSpec(f"{prefix}.experts.{e}.up_proj.weight", (spec.intermediate, spec.hidden)),
                          TensorSpec(f"{prefix}.experts.{e}.down_proj.weight", (spec.hidden, spec.intermediate))]
            return specs

        def __init__(self, spec, tensors, runtime):
            self.spec = spec
            act = runtime.precision.act
            self.router = tensors["router.weight"].to(runtime.device, torch.float32)
            take = lambda name: torch.stack([tensors[f"experts.{e}.{name}.weight"] for e in range(spec.experts)]).to(runtime.device, act)
            self.gate, self.up, self.down = take("gate_proj"), take("up_proj"), take("down_proj")

        def forward(self, x, ctx):
            # the step's flat token batch is the domain the tokens are sorted by expert in
            logits = x.float() @ self.router.T
            top_logits, chosen = logits.topk(self.spec.top, dim=-1)
            gates = torch.softmax(top_logits, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.spec.experts):
                rows, which = (chosen == e).nonzero(as_tuple=True)
                if rows.numel() == 0:
                    continue
                h = x[rows]
                act = torch.nn.functional.silu((h @ self.gate[e].T).float()).to(x.dtype) * (h @ self.up[e].T)
                out.index_add_(0, rows, (act @ self.down[e].T).float() * gates[rows, which][:, None])
            return out.to(x.dtype)


def plain_routed(h, w, prefix):
    logits = h @ w[f"{prefix}.router.weight"].T
    top_logits, chosen = logits.topk(TOP, dim=-1)
    gates = torch.softmax(top_logits, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(TOP):
            out[t] += gates[t, j] * plain.swiglu_mlp(h[t:t + 1], w, f"{prefix}.experts.{int(chosen[t, j])}")[0]
    return out


@pytest.mark.parametrize("dtype,tolerance", [("float32", 3e-5), ("bfloat16", 4e-2)])
def test_toy_model_with_a_routed_feed_forward(dtype, tolerance):
    from mrun_b200.config import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec
    from mrun_b200.engine import Executor, StepEntry
    from mrun_b200.weights import expected_tensors, random_tensors
    register_routed()
    norm = RMSNormSpec(HIDDEN, EPS)
    attention = AttentionSpec(HIDDEN, HEADS, KV_HEADS, HEAD_DIM, HEAD_DIM ** -0.5, RMSNormSpec(HEAD_DIM, EPS),
                              RotarySpec(HEAD_DIM, HEAD_DIM, THETA), None)
    layers = (LayerSpec("model.layers.0", attention, RoutedSpec(HIDDEN, 24, EXPERTS, TOP), norm, norm),
              LayerSpec("model.layers.1", attention, GatedMLPSpec(HIDDEN, INTER), norm, norm))
    spec = ModelSpec("ToyRoutedForCausalLM", VOCAB, HIDDEN, 512, layers, norm, tie_embeddings=True)
    names = {t.name for t in expected_tensors(spec)}
    assert "model.layers.0.mlp.experts.4.down_proj.weight" in names and "model.layers.1.mlp.gate_proj.weight" in names
    tensors = dict(random_tensors(spec, seed=5, std=0.08, norm_noise=0.1))
    w = {k: v.float() for k, v in tensors.items()}
    ex = Executor(spec, tensors, dtype=dtype, page_size=4, num_pages=64, max_requests=3)

    def plain_model(tokens):
        positions = torch.arange(len(tokens))
        x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
        rms = lambda x, name: plain.rms_norm(x, w[name], EPS)
        for i in range(2):
            a, _ = plain_attention(rms(x, f"model.layers.{i}.input_layernorm.weight"), w, f"model.layers.{i}.self_attn",
                                   positions, True, HEAD_DIM, 1.0, None)
            x = x + a
            h = rms(x, f"model.layers.{i}.post_attention_layernorm.weight")
            x = x + (plain_routed(h, w, "model.layers.0.mlp") if i == 0 else plain.swiglu_mlp(h, w, "model.layers.1.mlp"))
        return rms(x, "model.norm.weight") @ w["model.embed_tokens.weight"].T

    gen = torch.Generator().manual_seed(4)
    seqs = {name: torch.randint(0, VOCAB, (n,), generator=gen).tolist() for name, n in (("a", 45), ("b", 23))}
    want = {name: plain_model(tokens) for name, tokens in seqs.items()}
    scale = max(float(x.abs().max()) for x in want.values())

    def check(name, start, logits):
        got = logits.cpu()
        # a near-tie between two experts may fall the other way in bfloat16: such rows are rare
        # and would show as a large error in one row, which the tolerance does not hide
        error = float((got - want[name][start:start + got.shape[0]]).abs().max()) / scale
        assert error <= tolerance, (name, start, error)

    r = ex.admit("whole")
    check("a", 0, ex.step([StepEntry(r, seqs["a"], range(45))]))
    ex.release(r)
    live = {name: ex.admit(name) for name in seqs}
    fed = {name: 0 for name in seqs}
    sizes = {"a": [20, 1, 1, 2, 21], "b": [1, 1, 19, 1, 1]}
    for turn in range(5):
        entries, parts = [], []
        for name in seqs:
            n = sizes[name][turn]
            entries.append(StepEntry(live[name], seqs[name][fed[name]:fed[name] + n], range(n)))
            parts.append((name, fed[name], n))
            fed[name] += n
        logits = ex.step(entries)
        row = 0
        for name, start, n in parts:
            check(name, start, logits[row:row + n])
            row += n
    for request in live.values():
        ex.release(request)
    ex.cache.check_invariants()


# ------------------------------------------------------------------ hooks of the model, biases, another gate function

@dataclass(frozen=True)
class ScaleSpec:
    """x * factor (a scale of the embedding)."""
    kind: ClassVar[str] = "toy_scale"
    factor: float


@dataclass(frozen=True)
class SoftCapSpec:
    """cap * tanh(x / cap) + bias (a soft cap and a bias of the logits; the bias is a checkpoint tensor)."""
    kind: ClassVar[str] = "toy_soft_cap"
    cap: float
    size: int
    prefix: str = "logits_cap"


@dataclass(frozen=True)
class TokenLinearSpec:
    """y = x W^T, token by token: a mixer without a cache that knows nothing of pending products."""
    kind: ClassVar[str] = "toy_token_linear"
    hidden: int


def register_hooks():
    from mrun_b200.config import TensorSpec
    from mrun_b200.parts import TRANSFORMS, register_mixer, register_transform
    if "toy_scale" in TRANSFORMS.kinds():
        return

    @register_transform("toy_scale")
    class Scale:
        @staticmethod
        def tensor_specs(spec, prefix):
            return []

        def __init__(self, spec, tensors, runtime):
            self.factor = spec.factor

        def forward(self, x):
            return x.mul_(self.factor)

    @register_transform("toy_soft_cap")
    class SoftCap:
        @staticmethod
        def tensor_specs(spec, prefix):
            return [TensorSpec(f"{prefix}.bias", (spec.size,))]

        def __init__(self, spec, tensors, runtime):
            self.cap = spec.cap
            self.bias = tensors["bias"].to(runtime.device, torch.float32)

        def forward(self, logits):
            return torch.tanh(logits / self.cap) * self.cap + self.bias

    @register_mixer("toy_token_linear")
    class TokenLinear:
        graph_safe = True

        @staticmethod
        def tensor_specs(spec, prefix):
            return [TensorSpec(f"{prefix}.proj.weight", (spec.hidden, spec.hidden))]

        def __init__(self, spec, tensors, runtime):
            self.weight = runtime.matrix(tensors["proj.weight"])

        def cache_need(self):
            return None

        def forward(self, x, ctx, cache):
            assert isinstance(x, torch.Tensor)            # normed rows are finished for a part like this one
            return (x.float() @ self.weight.float().T).to(x.dtype)


@pytest.mark.parametrize("dtype,tolerance", [("float32", 3e-5), ("bfloat16", 4e-2)])
def test_model_hooks_biases_and_another_gate_function(dtype, tolerance):
    """An embedding scale and a logit soft cap with a bias as transforms of the model spec, linear
    layers with biases in the checkpoint, a tanh-GELU gate, and a toy mixer between product norms
    (it gets plain tensors where a product part would get rows with a pending scale): nothing of
    it edits the framework.  Whole, in portions, and token by token through the captured step."""
    import math
    from mrun_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec)
    from mrun_b200.engine import Executor, StepEntry
    from mrun_b200.weights import bind_tensors, random_tensors
    register_hooks()
    hidden, heads, kv_heads, head_dim, inter, vocab, eps, theta = 64, 4, 2, 32, 96, 211, 1e-5, 1e4
    norm = RMSNormSpec(hidden, eps)
    mlp = GatedMLPSpec(hidden, inter, activation="gelu_tanh")
    attn = AttentionSpec(hidden, heads, kv_heads, head_dim, head_dim ** -0.5, RMSNormSpec(head_dim, eps),
                         RotarySpec(head_dim, head_dim, theta), None)
    layers = (LayerSpec("model.layers.0", attn, mlp, norm, norm),
              LayerSpec("model.layers.1", TokenLinearSpec(hidden), mlp, norm, norm, mixer_prefix="mix"),
              LayerSpec("model.layers.2", attn, mlp, norm, norm))
    spec = ModelSpec("ToyHooksForCausalLM", vocab, hidden, 512, layers, norm, tie_embeddings=True,
                     embedding_transform=ScaleSpec(math.sqrt(hidden)), logits_transform=SoftCapSpec(4.0, vocab))
    tensors = dict(random_tensors(spec, seed=5, std=0.08, norm_noise=0.1))
    assert "logits_cap.bias" in tensors and not any(n.endswith("proj.bias") for n in tensors)
    gen = torch.Generator().manual_seed(2)
    bias = lambda n: (torch.randn(n, generator=gen) * 0.3).to(torch.bfloat16)
    for i in (0, 2):
        p = f"model.layers.{i}"
        tensors[f"{p}.self_attn.q_proj.bias"] = bias(heads * head_dim)
        tensors[f"{p}.self_attn.v_proj.bias"] = bias(kv_heads * head_dim)
        tensors[f"{p}.self_attn.o_proj.bias"] = bias(hidden)
        tensors[f"{p}.mlp.up_proj.bias"] = bias(inter)
    tensors["model.layers.1.mlp.down_proj.bias"] = bias(hidden)
    tensors = bind_tensors(spec, tensors)
    w = {k: v.float() for k, v in tensors.items()}

    def plain_model(tokens):
        positions = torch.arange(len(tokens))
        x = w["model.embed_tokens.weight"][torch.tensor(tokens)] * math.sqrt(hidden)
        n = lambda t, name: plain.rms_norm(t, w[name], eps)
        b = lambda name, size: w.get(name, torch.zeros(size))
        for i in range(3):
            p = f"model.layers.{i}"
            h = n(x, f"{p}.input_layernorm.weight")
            if i == 1:
                a = h @ w[f"{p}.mix.proj.weight"].T
            else:
                q = (h @ w[f"{p}.self_attn.q_proj.weight"].T + b(f"{p}.self_attn.q_proj.bias", 1)).view(-1, heads, head_dim)
                k = (h @ w[f"{p}.self_attn.k_proj.weight"].T).view(-1, kv_heads, head_dim)
                v = (h @ w[f"{p}.self_attn.v_proj.weight"].T + b(f"{p}.self_attn.v_proj.bias", 1)).view(-1, kv_heads, head_dim)
                q = plain.rope(plain.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], eps), positions, theta)
                k = plain.rope(plain.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], eps), positions, theta)
                o = plain.attention_scores_softmax_values(q, k, v, head_dim ** -0.5, positions, None)
                a = o.reshape(-1, heads * head_dim) @ w[f"{p}.self_attn.o_proj.weight"].T + b(f"{p}.self_attn.o_proj.bias", 1)
            x = x + a
            h = n(x, f"{p}.post_attention_layernorm.weight")
            g = h @ w[f"{p}.mlp.gate_proj.weight"].T
            u = h @ w[f"{p}.mlp.up_proj.weight"].T + b(f"{p}.mlp.up_proj.bias", 1)
            act = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u
            x = x + act @ w[f"{p}.mlp.down_proj.weight"].T + b(f"{p}.mlp.down_proj.bias", 1)
        logits = n(x, "model.norm.weight") @ w["model.embed_tokens.weight"].T
        return torch.tanh(logits / 4.0) * 4.0 + w["logits_cap.bias"]

    ex = Executor(spec, tensors, dtype=dtype, page_size=8, num_pages=64, max_requests=4)
    assert ex.model.graph_safe
    tokens = torch.randint(0, vocab, (70,), generator=gen).tolist()
    want = plain_model(tokens)
    scale = float(want.abs().max())

    def check(start, logits):
        got = logits.float().cpu()
        error = float((got - want[start:start + got.shape[0]]).abs().max()) / scale
        assert error <= tolerance, (dtype, start, error)

    r = ex.admit("whole")
    check(0, ex.step([StepEntry(r, tokens, range(70))]))
    ex.release(r)
    r = ex.admit("portions")
    at = 0
    for n_tokens in (33, 2, 9, 1, 1, 5):                      # 33 rows: the vendor GEMM; the rest: the decode GEMM
        check(at, ex.step([StepEntry(r, tokens[at:at + n_tokens], range(n_tokens))]))
        at += n_tokens
    for i in range(at, 70):                                   # the captured step
        entries = [StepEntry(r, [tokens[i]], [0])]
        ex.decode_step(entries)
        check(i, ex.decode_logits(entries))
    ex.release(r)
    ex.cache.check_invariants()
