"""One registry from an architecture's name to its typed config and its builder.

The name is the first entry of ``architectures`` in ``config.json``
(``"Qwen2ForCausalLM"``); a checkpoint without that key is matched by ``model_type``.
The builder turns the typed config into a ``DecoderSpec``: which parts, with which
sizes, in which order, reading which checkpoint tensors.  Adding an architecture is one
``register_architecture`` call; nothing else in the package names a model.

(The reference has no such table: ``emberserve/config.py:122`` lists model types and
``emberserve/model/weights.py:257-263`` switches on the config.)
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable

from emberserve_b200.config.model import ConfigError, ModelConfig, read_config_json
from emberserve_b200.parts.decoder import Decoder, DecoderSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type[ModelConfig]
    build_spec: Callable[[Any], DecoderSpec]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type[ModelConfig],
                          build_spec: Callable[[Any], DecoderSpec],
                          model_types: tuple[str, ...] = ()) -> Architecture:
    arch = Architecture(name, config_cls, build_spec, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(cfg: dict[str, Any]) -> Architecture:
    """The architecture that serves a ``config.json`` dict."""
    _ensure_builtin()
    names = cfg.get("architectures") or []
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = cfg.get("model_type")
    if not names and model_type is not None:
        for arch in _ARCHITECTURES.values():
            if model_type in arch.model_types:
                return arch
    raise ConfigError(f"unsupported architecture {names or model_type!r}; "
                      f"supported: {registered_architectures()}")


def load_config(model_dir: str | os.PathLike) -> ModelConfig:
    cfg = read_config_json(model_dir)
    return resolve_architecture(cfg).config_cls.from_dict(cfg)


def architecture_of(config: ModelConfig) -> Architecture:
    _ensure_builtin()
    for arch in _ARCHITECTURES.values():
        if type(config) is arch.config_cls:
            return arch
    raise ConfigError(f"no architecture is registered for {type(config).__name__}")


def build_decoder(config: ModelConfig) -> Decoder:
    """The model of `config`, without weights."""
    return Decoder(architecture_of(config).build_spec(config))


def _ensure_builtin() -> None:
    import emberserve_b200.models  # noqa: F401  (registers the built-in architecture)
