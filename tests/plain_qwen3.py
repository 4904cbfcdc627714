"""A plain, slow Qwen3 dense decoder: whole sequences, no cache, 32-bit on the CPU, one function
per part.  It shares no code with ``mrun_b200``: it reads the model folder with the ``safetensors``
package and computes with plain torch tensor arithmetic.

It rests on the reference's formulas, each cited by file:line within hupe1980/mrun.  The
reference's own model code cannot be built or imported here (no Rust toolchain, its array library
is an unvendored crates.io dependency, its Python scripts need mlx), so there is no recorded output
of the reference to compare with.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------- loading

def load_folder(model_dir: str):
    """config.json as a dict and every tensor widened to float32."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    for name in sorted(os.listdir(model_dir)):
        if name.endswith(".safetensors"):
            for key, value in load_file(os.path.join(model_dir, name)).items():
                weights[key] = value.to(torch.float32)
    return cfg, weights


def head_dim_of(cfg: dict) -> int:
    # crates/mrun-engine/src/models/qwen3.rs:40-42: head_dim, else hidden / heads
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def rope_theta_of(cfg: dict) -> float:
    # crates/mrun-engine/src/models/qwen3.rs:43-47: rope_parameters.rope_theta, else rope_theta
    rope = cfg.get("rope_parameters")
    if isinstance(rope, dict) and "rope_theta" in rope:
        return float(rope["rope_theta"])
    return float(cfg["rope_theta"])


# --------------------------------------------------------------------------- parts

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2, last axis) + eps) * w.
    crates/mrun-engine/src/load.rs:348-364 (the call); crates/mrun-engine/src/models/gated_delta.rs:11-13
    (eps is added to the mean of squares)."""
    ms = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: Optional[int] = None) -> torch.Tensor:
    """x: [L, n, D]; pair (j, j + rd/2), angle = p * theta^(-2j/rd), angle in 64-bit.
    crates/mrun-engine/src/models/common.rs:215-230 (non-traditional = half split, base theta,
    scale 1), crates/mrun-engine/src/models/common.rs:264-280 (angle in f64, rotation formulas)."""
    d = x.shape[-1]
    rd = d if rotary_dim is None else rotary_dim
    half = rd // 2
    j = torch.arange(half, dtype=torch.float64)
    inv = torch.tensor(theta, dtype=torch.float64) ** (-2.0 * j / rd)
    angle = positions.to(torch.float64)[:, None] * inv[None, :]          # [L, half]
    cos = angle.cos().to(torch.float32)[:, None, :]
    sin = angle.sin().to(torch.float32)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rd]
    out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., rd:]], dim=-1)
    return out


def attention_scores_softmax_values(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                                    q_positions: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """q: [L, nh, D]; k, v: [S, nkv, D] for key positions 0..S-1.  Query head h reads kv head
    h // (nh / nkv); a query at position p sees keys 0..p (window W: p-W+1..p); softmax in 32-bit.
    crates/mrun-engine/src/models/common.rs:129 (scale), :199-205 (causal when L > 1, sdpa call),
    crates/mrun-engine/src/tensor/nuvec.rs:866-872 (causal mask aligned to the end of the keys)."""
    L, nh, D = q.shape
    S, nkv, _ = k.shape
    group = nh // nkv
    out = torch.empty_like(q)
    key_pos = torch.arange(S)
    for h in range(nh):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale                          # [L, S]
        visible = key_pos[None, :] <= q_positions[:, None]
        if window is not None:
            visible &= key_pos[None, :] > (q_positions[:, None] - window)
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    positions: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """Projections, per-head q/k norm, rope, attention, output projection.
    crates/mrun-engine/src/models/common.rs:165-171 (three projections, y = x W^T,
    crates/mrun-engine/src/load.rs:294-306), :183,194-196 (per-head RMSNorm of q and k before
    rope; v untouched), :197 (rope on q and k), :206,137 (heads concatenated, o_proj)."""
    nh, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    eps = cfg["rms_norm_eps"]
    L = h.shape[0]
    q = (h @ w[f"{prefix}.q_proj.weight"].T).view(L, nh, D)
    k = (h @ w[f"{prefix}.k_proj.weight"].T).view(L, nkv, D)
    v = (h @ w[f"{prefix}.v_proj.weight"].T).view(L, nkv, D)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    theta = rope_theta_of(cfg)
    q, k = rope(q, positions, theta), rope(k, positions, theta)
    o = attention_scores_softmax_values(q, k, v, float(D) ** -0.5, positions, window)
    return o.reshape(L, nh * D) @ w[f"{prefix}.o_proj.weight"].T


def swiglu_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), silu(z) = z * sigmoid(z).
    crates/mrun-engine/src/models/common.rs:329-339, crates/mrun-engine/src/models/activations.rs:46-59."""
    gate = h @ w[f"{prefix}.gate_proj.weight"].T
    up = h @ w[f"{prefix}.up_proj.weight"].T
    return (gate * torch.sigmoid(gate) * up) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict,
                  positions: torch.Tensor) -> torch.Tensor:
    """x + attn(norm(x)), then x + mlp(norm(x)).  crates/mrun-engine/src/models/qwen3.rs:133-145."""
    p = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    x = x + attention_block(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", cfg, positions)
    x = x + swiglu_mlp(rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [L, vocab] of a whole sequence at positions 0..L-1.
    Embedding crates/mrun-engine/src/load.rs:330-335; final norm and head (tied: the embedding
    table) crates/mrun-engine/src/models/common.rs:382-392, crates/mrun-engine/src/load.rs:338-343."""
    ids = torch.tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["model.embed_tokens.weight"][ids]
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions)
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return h @ head.T


# --------------------------------------------------------------------------- sampling

_M64 = (1 << 64) - 1


def mix64(z: int) -> int:
    """SplitMix64's finaliser on a 64-bit integer (the engine's counter-based generator)."""
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def draw_key(seed: int, draw: int) -> int:
    """Key of the draw-th token of a request (draws count from 1):
    seed * 0x9E3779B97F4A7C15 + draw, crates/mrun-engine/src/nuvec_engine.rs:224-231; mixed once
    more so that neighbouring draws share no structure."""
    return mix64((seed * 0x9E3779B97F4A7C15 + draw) & _M64)


def gumbel_noise(key: int, vocab: int) -> np.ndarray:
    idx = np.arange(vocab, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(key) + idx
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = ((z >> np.uint64(40)).astype(np.float64) + 0.5) / 16777216.0
    return (-np.log(-np.log(u))).astype(np.float32)


def filter_threshold(logits: np.ndarray, top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0) -> np.ndarray:
    """Boolean keep-mask after top-p, then min-p, then top-k
    (crates/mrun-engine/src/sample.rs:38-78, order at :121-129)."""
    x = logits.astype(np.float64)
    lp = x - (np.log(np.sum(np.exp(x - x.max()))) + x.max())
    keep = np.ones_like(lp, dtype=bool)
    if 0.0 < top_p < 1.0:
        order = np.argsort(lp, kind="stable")                 # ascending
        probs = np.exp(lp[order])
        above = np.concatenate([np.cumsum(probs[::-1])[::-1][1:], [0.0]])   # mass strictly after
        total = above[0] + probs[0]
        dropped = int(np.sum(above >= total * top_p))
        keep &= lp >= lp[order][dropped]
    if min_p > 0.0:
        keep &= lp >= lp.max() + math.log(min_p)
    if top_k > 0 and top_k < len(lp):
        kth = np.sort(lp)[::-1][top_k - 1]
        keep &= lp >= kth
    return keep


def sample_token(logits: np.ndarray, temperature: float, key: int = 0, top_p: float = 1.0,
                 top_k: int = 0, min_p: float = 0.0) -> int:
    """Greedy at temperature 0 (crates/mrun-engine/src/sample.rs:118-120), else a categorical
    draw from the kept tokens at 1/temperature (:130-132) by the Gumbel-max rule."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature == 0.0:
        return int(np.argmax(logits))
    keep = filter_threshold(logits, top_p, top_k, min_p)
    score = logits * np.float32(1.0 / np.float32(temperature)) + gumbel_noise(key, len(logits))
    score = np.where(keep, score, -np.inf)
    return int(np.argmax(score))


def top_logprobs(logits: np.ndarray, n: int) -> List[tuple]:
    """crates/mrun-engine/src/sample.rs:134-156: the n most likely tokens with lp = logits -
    logsumexp(logits) (sample.rs:10-13), most likely first, ties by the smaller id."""
    logits = np.asarray(logits, dtype=np.float64)
    lp = logits - (logits.max() + np.log(np.exp(logits - logits.max()).sum()))
    order = sorted(range(len(lp)), key=lambda i: (-lp[i], i))[:max(1, min(n, len(lp)))]
    return [(i, float(lp[i])) for i in order]


def apply_token_mask(logits: np.ndarray, allowed: Sequence[int]) -> np.ndarray:
    """crates/mrun-engine/src/sample.rs:104-116: where(mask, logprobs, -inf); the log-sum-exp it
    subtracts before is one constant a row, so the filters and the draw after it (which look at
    differences among the allowed tokens) see the same on masked logits."""
    out = np.full(len(logits), -np.inf, dtype=np.float32)
    allowed = [i for i in allowed if 0 <= i < len(logits)]
    out[allowed] = np.asarray(logits, dtype=np.float32)[allowed]
    return out


def apply_repetition_penalty(logits: np.ndarray, recent: Sequence[int], penalty: float) -> np.ndarray:
    """crates/mrun-engine/src/sample.rs:23-36: logits of recent ids divided by the penalty when
    >= 0, multiplied when negative."""
    out = np.array(logits, dtype=np.float32)
    for token in set(recent):
        out[token] = out[token] / penalty if out[token] >= 0 else out[token] * penalty
    return out


def generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], max_tokens: int,
             temperature: float = 0.0, seed: int = 0, eos: Sequence[int] = ()) -> List[int]:
    """Recomputes the whole sequence for every token."""
    tokens = list(prompt)
    out: List[int] = []
    for n in range(1, max_tokens + 1):
        logits = forward(cfg, w, tokens)[-1].numpy()
        token = sample_token(logits, temperature, draw_key(seed, n))
        out.append(token)
        tokens.append(token)
        if token in eos:
            break
    return out
