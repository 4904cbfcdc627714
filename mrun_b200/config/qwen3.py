"""Typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

Keys, defaults and refusals follow the reference:
crates/mrun-engine/src/models/qwen3.rs:37-74 (attention settings, rope, tied head),
crates/mrun-engine/src/models/registry.rs:108-160 (layout keys),
crates/mrun-engine/src/models/registry.rs:208-231 (``layer_types``),
crates/mrun-engine/src/models/registry.rs:250-259 (``torch_dtype``),
crates/mrun-engine/src/models/common.rs:30-46 (rope scaling types).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, eos_token_ids, opt_bool, opt_int, req_int, req_num
from .spec import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec)


@dataclass(frozen=True)
class Qwen3Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    eos_token_id: Tuple[int, ...] = ()

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any], model_dir: Optional[str] = None) -> "Qwen3Config":
        layers = req_int(cfg, "num_hidden_layers")
        hidden = req_int(cfg, "hidden_size")
        heads = req_int(cfg, "num_attention_heads")
        kv_heads = req_int(cfg, "num_key_value_heads")
        head_dim = opt_int(cfg, "head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("head_dim", "is missing and hidden_size is not a multiple of "
                                  "num_attention_heads")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError("num_key_value_heads",
                              f"({kv_heads}) does not divide num_attention_heads ({heads})")
        if head_dim % 2:
            raise ConfigError("head_dim", f"must be even for rotary positions, got {head_dim}")

        rope = cfg.get("rope_parameters")
        rope = rope if isinstance(rope, dict) else None
        theta = None
        if rope is not None and isinstance(rope.get("rope_theta"), (int, float)):
            theta = float(rope["rope_theta"])
        elif isinstance(cfg.get("rope_theta"), (int, float)) and not isinstance(cfg.get("rope_theta"), bool):
            theta = float(cfg["rope_theta"])
        if theta is None:
            raise ConfigError("rope_theta", "is missing")
        if theta <= 0:
            raise ConfigError("rope_theta", f"must be positive, got {theta}")
        scaling = rope if rope is not None else cfg.get("rope_scaling")
        if isinstance(scaling, dict):
            kind = scaling.get("type") or scaling.get("rope_type") or "default"
            if kind == "linear":
                factor = req_num(scaling, "factor")
                if factor != 1.0:
                    raise ConfigError("rope_scaling", "only the default RoPE is supported")
            elif kind != "default":
                raise ConfigError("rope_scaling", f"type {kind} is not supported")

        types = cfg.get("layer_types")
        if isinstance(types, list):
            if len(types) != layers:
                raise ConfigError("layer_types", f"has {len(types)} entries for {layers} layers")
            for kind in types:
                if kind != "full_attention":
                    raise ConfigError("layer_types", f"has unknown entry {kind!r}")

        dtype = cfg.get("torch_dtype", cfg.get("dtype"))
        if dtype is None:
            dtype = "bfloat16"
        if dtype not in ("bfloat16", "float16", "float32"):
            raise ConfigError("torch_dtype", f"{dtype} is not supported")
        for key in ("quantization", "quantization_config"):
            if cfg.get(key) is not None:
                raise ConfigError(key, "is set: quantized weights are not supported")

        eps = req_num(cfg, "rms_norm_eps")
        if not eps > 0:
            raise ConfigError("rms_norm_eps", f"must be positive, got {eps}")
        return cls(
            num_hidden_layers=layers,
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=req_int(cfg, "intermediate_size"),
            vocab_size=req_int(cfg, "vocab_size"),
            max_position_embeddings=req_int(cfg, "max_position_embeddings"),
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=opt_bool(cfg, "tie_word_embeddings", False),
            torch_dtype=dtype,
            eos_token_id=eos_token_ids(model_dir, cfg),
        )

    def to_dict(self) -> dict:
        """config.json contents that :meth:`from_dict` reads back to an equal configuration."""
        out = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    # ------------------------------------------------------------------ derived
    def kv_bytes_per_token(self, bytes_per_element: int = 2) -> int:
        """K and V bytes of one token over all layers
        (crates/mrun-engine/src/models/registry.rs:157)."""
        return (self.num_hidden_layers * 2 * self.num_key_value_heads * self.head_dim
                * bytes_per_element)

    def num_parameters(self) -> int:
        h, d = self.hidden_size, self.head_dim
        attn = (self.num_attention_heads + 2 * self.num_key_value_heads) * d * h \
            + self.num_attention_heads * d * h + 2 * d
        mlp = 3 * h * self.intermediate_size
        layer = attn + mlp + 2 * h
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.num_hidden_layers * layer + self.vocab_size * h + head + h

    def to_spec(self) -> ModelSpec:
        """The parts of this architecture, layer by layer
        (crates/mrun-engine/src/models/qwen3.rs:69-117, 133-145)."""
        eps = self.rms_norm_eps
        attention = AttentionSpec(
            hidden=self.hidden_size,
            heads=self.num_attention_heads,
            kv_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            # crates/mrun-engine/src/models/common.rs:129
            softmax_scale=float(self.head_dim) ** -0.5,
            qk_norm=RMSNormSpec(self.head_dim, eps),
            # rope over the whole head, crates/mrun-engine/src/models/qwen3.rs:59
            position=RotarySpec(self.head_dim, self.head_dim, self.rope_theta),
            window=None,
        )
        mlp = GatedMLPSpec(self.hidden_size, self.intermediate_size, "silu")
        norm = RMSNormSpec(self.hidden_size, eps)
        layers = tuple(
            LayerSpec(prefix=f"model.layers.{i}", mixer=attention, feed_forward=mlp,
                      mixer_norm=norm, feed_forward_norm=norm)
            for i in range(self.num_hidden_layers))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            layers=layers,
            final_norm=norm,
            tie_embeddings=self.tie_word_embeddings,
            eos_token_ids=self.eos_token_id,
        )
