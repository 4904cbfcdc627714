"""One registry from an architecture's name to its configuration class.

``config.json`` chooses the model everywhere in the framework: by ``architectures[0]`` or by
``model_type`` (the reference keys its table by ``model_type``,
crates/mrun-engine/src/models/registry.rs:36-80, and lists the supported families in the
error, crates/mrun-engine/src/models/mod.rs:288-303).

A configuration class has ``architecture`` and ``model_type`` attributes, a
``from_dict(config, model_dir)`` constructor, ``to_dict()`` and ``to_spec()`` returning a
:class:`mrun_b200.config.spec.ModelSpec`.
"""
from __future__ import annotations

import os
from typing import Any, Mapping, Optional

from .config.base import ConfigError, UnsupportedArchitecture, read_json

_BY_ARCHITECTURE: dict[str, type] = {}
_BY_MODEL_TYPE: dict[str, type] = {}


def register_architecture(config_cls: type) -> type:
    """Adds a configuration class under its ``architecture`` and ``model_type`` names."""
    for attr in ("architecture", "model_type", "from_dict", "to_spec"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"{config_cls.__name__} lacks {attr}")
    _BY_ARCHITECTURE[config_cls.architecture] = config_cls
    _BY_MODEL_TYPE[config_cls.model_type] = config_cls
    return config_cls


def supported() -> list[str]:
    return sorted(_BY_MODEL_TYPE)


def resolve(cfg: Mapping[str, Any], where: Optional[str] = None) -> type:
    """The configuration class that ``cfg`` names."""
    architectures = cfg.get("architectures")
    if isinstance(architectures, list):
        for name in architectures:
            if name in _BY_ARCHITECTURE:
                return _BY_ARCHITECTURE[name]
    model_type = cfg.get("model_type")
    if isinstance(model_type, str) and model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    if not isinstance(model_type, str):
        if isinstance(architectures, list) and architectures:
            raise UnsupportedArchitecture(str(architectures[0]), supported(), where)
        raise ConfigError("model_type", "is missing")
    raise UnsupportedArchitecture(model_type, supported(), where)


def load_config(model_dir: str):
    """Reads ``model_dir/config.json`` into the typed configuration of its architecture."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{model_dir} has no config.json")
    cfg = read_json(path)
    return resolve(cfg, model_dir).from_dict(cfg, model_dir)


def _register_builtin() -> None:
    from .config.qwen3 import Qwen3Config
    register_architecture(Qwen3Config)


_register_builtin()
