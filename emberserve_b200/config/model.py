"""Typed model configurations, read from an architecture's own ``config.json`` keys.

``Qwen2Config`` carries every number the Qwen2.5 dense decoder needs.  Nothing in
the package hard-codes a size: parts receive their sizes from here through the
architecture's builder (``emberserve_b200/models/qwen2.py``).

Parity with the reference: ``emberserve/config.py:90-110`` (fields),
``config.py:169-234`` (``from_hf_dir``: required keys, defaults of optional keys,
refusals).  One deliberate extension: the reference refuses a checkpoint whose
``use_sliding_window`` is true (``config.py:177-178``); here the three Qwen2 keys
``sliding_window`` / ``use_sliding_window`` / ``max_window_layers`` are honoured,
so that layers of one model may differ in their cache needs.
"""

from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A ``config.json`` that this engine cannot serve, with the reason."""


def read_config_json(model_dir: str | os.PathLike) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    return json.loads(path.read_text())


@dataclass(frozen=True)
class ModelConfig:
    """Base of all typed architecture configs.  A subclass names the ``config.json``
    ``architectures`` entry it serves and parses that architecture's keys."""

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        raise NotImplementedError

    def save(self, model_dir: str | os.PathLike) -> None:
        Path(model_dir).mkdir(parents=True, exist_ok=True)
        (Path(model_dir) / "config.json").write_text(json.dumps(self.to_dict(), indent=1) + "\n")


def _require(cfg: dict[str, Any], key: str, kind: type) -> Any:
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"config.json lacks the required key {key!r}")
    value = cfg[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json key {key!r} must be an integer, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """Qwen2 / Qwen2.5 dense decoder (``Qwen2ForCausalLM``).

    Keys and defaults follow ``emberserve/config.py:202-234``: the first five are
    required; ``num_key_value_heads`` defaults to the head count, ``head_dim`` to
    ``hidden_size // num_attention_heads`` (``config.py:131-132``), ``rms_norm_eps``
    to 1e-6, ``rope_theta`` to 1e6, ``tie_word_embeddings`` and ``attention_bias`` to
    true for ``model_type == "qwen2"``, ``eos_token_id`` to 151645 (``config.py:186-194``).
    """

    architecture: ClassVar[str] = "Qwen2ForCausalLM"

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    attention_bias: bool
    eos_token_ids: tuple[int, ...]
    bos_token_id: int | None = None
    # Sliding-window attention: layers with index >= max_window_layers attend to the
    # last `sliding_window` keys only (their own position included).  None = off.
    sliding_window: int | None = None
    max_window_layers: int = 0

    def __post_init__(self) -> None:
        def positive(name: str) -> None:
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")

        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "max_position_embeddings"):
            positive(name)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary encoding")
        if not self.eos_token_ids:
            raise ConfigError("config.json has no eos_token_id")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError(f"sliding_window must be positive, got {self.sliding_window}")
        if not (self.rms_norm_eps > 0 and self.rope_theta > 0):
            raise ConfigError("rms_norm_eps and rope_theta must be positive")

    # ---- derived ---------------------------------------------------------------------
    @property
    def num_kv_groups(self) -> int:
        """Query heads per KV head (``config.py:156-159``)."""
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def eos_token_id(self) -> int:
        return self.eos_token_ids[0]

    def layer_window(self, layer_idx: int) -> int | None:
        """Window of layer `layer_idx`: None where it attends to all keys."""
        if self.sliding_window is None or layer_idx < self.max_window_layers:
            return None
        return self.sliding_window

    def kv_bytes_per_token(self, element_size: int) -> int:
        """Cache bytes per token over all layers (``config.py:161-167``)."""
        return (2 * self.num_hidden_layers * self.num_key_value_heads * self.head_dim
                * element_size)

    def num_parameters(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        per_layer = h * (q + 2 * kv) + q * h + 3 * h * i + 2 * h
        if self.attention_bias:
            per_layer += q + 2 * kv
        total = self.num_hidden_layers * per_layer + v * h + h
        if not self.tie_word_embeddings:
            total += v * h
        return total

    # ---- config.json -----------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "Qwen2Config":
        model_type = cfg.get("model_type", "qwen2")
        if model_type != "qwen2":
            raise ConfigError(f"Qwen2Config serves model_type 'qwen2', got {model_type!r}")
        if cfg.get("mlp_bias", False):
            raise ConfigError("mlp_bias=True is not supported")  # config.py:179-180
        rope_scaling = cfg.get("rope_scaling")
        if rope_scaling is not None:  # config.py:195-201
            kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
            if kind != "default":
                raise ConfigError(f"unsupported rope_scaling type {kind!r}")
        eos = cfg.get("eos_token_id", 151645)
        if isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (int(eos),)
        else:
            raise ConfigError(f"eos_token_id must be an integer or a list, got {eos!r}")
        heads = _require(cfg, "num_attention_heads", int)
        hidden = _require(cfg, "hidden_size", int)
        head_dim = cfg.get("head_dim") or hidden // heads
        layers = _require(cfg, "num_hidden_layers", int)
        window = cfg.get("sliding_window")
        if window in (None, 0) or not cfg.get("use_sliding_window", True):
            window = None
        bos = cfg.get("bos_token_id")
        return cls(
            vocab_size=_require(cfg, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_require(cfg, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 32768)),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
            rope_theta=float(cfg.get("rope_theta", 1_000_000.0)),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", True)),
            attention_bias=bool(cfg.get("attention_bias", True)),
            eos_token_ids=eos_ids,
            bos_token_id=None if bos is None else int(bos),
            sliding_window=None if window is None else int(window),
            max_window_layers=int(cfg.get("max_window_layers", layers)) if window else 0,
        )

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "eos_token_id": (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                             else list(self.eos_token_ids)),
            "hidden_act": "silu",
            "use_sliding_window": self.sliding_window is not None,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
            d["max_window_layers"] = self.max_window_layers
        return d

    def replace(self, **changes: Any) -> "Qwen2Config":
        return dataclasses.replace(self, **changes)
