"""Helpers for reading a parsed ``config.json``.

Every reader names the key it could not use, in the reference's wording
("invalid config.json: <key> <reason>", crates/mrun-engine/src/models/mod.rs:274-275,
crates/mrun-engine/src/models/common.rs:14-26).
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used: names the key and the reason."""

    def __init__(self, key: str, reason: str):
        self.key = key
        self.reason = reason
        super().__init__(f"invalid config.json: {key} {reason}")


class UnsupportedArchitecture(ValueError):
    """config.json names an architecture that no registered model covers."""

    def __init__(self, name: str, supported: list[str], where: Optional[str] = None):
        self.name = name
        self.supported = list(supported)
        location = f" in {where}" if where else ""
        super().__init__(
            f"unsupported architecture '{name}'{location}\n"
            f"  supported families: {', '.join(sorted(supported))}"
        )


def read_json(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        value = json.load(f)
    if not isinstance(value, dict):
        raise ConfigError(os.path.basename(path), "is not a JSON object")
    return value


def req_int(cfg: Mapping[str, Any], key: str, minimum: int = 1) -> int:
    value = cfg.get(key)
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(key, "is missing or not an integer")
    if value < minimum:
        raise ConfigError(key, f"must be at least {minimum}, got {value}")
    return value


def opt_int(cfg: Mapping[str, Any], key: str, minimum: int = 1) -> Optional[int]:
    if cfg.get(key) is None:
        return None
    return req_int(cfg, key, minimum)


def req_num(cfg: Mapping[str, Any], key: str) -> float:
    value = cfg.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(key, "is missing or not a number")
    return float(value)


def opt_bool(cfg: Mapping[str, Any], key: str, default: bool) -> bool:
    value = cfg.get(key)
    if value is None:
        return default
    if not isinstance(value, bool):
        raise ConfigError(key, "is not a boolean")
    return value


def eos_token_ids(model_dir: Optional[str], cfg: Mapping[str, Any]) -> tuple[int, ...]:
    """Union of ``eos_token_id`` (int or list) from config.json and generation_config.json.

    The reference also maps the tokenizer's EOS text to an id
    (crates/mrun-engine/src/identity.rs:135-163); this engine takes token ids only and has
    no tokenizer, so only the numeric sources are read.
    """
    ids: set[int] = set()

    def take(value: Any) -> None:
        items = value if isinstance(value, list) else [value]
        for item in items:
            if isinstance(item, int) and not isinstance(item, bool) and item >= 0:
                ids.add(item)

    take(cfg.get("eos_token_id"))
    if model_dir is not None:
        path = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(path):
            try:
                take(read_json(path).get("eos_token_id"))
            except (OSError, ValueError):
                pass
    return tuple(sorted(ids))
