"""Typed model configurations read from an architecture's own config.json keys.

The reference has no configuration code of its own: it reads attributes of the object the
checkpoint loader builds (ampere_kv/runner.py:33-44: ``head_dim``, ``rope_theta``,
``hidden_act``, per-layer ``sliding_window``, per-norm ``variance_epsilon``; runner.py:321
``num_key_value_heads``; runner.py:331 ``eos_token_id``).  Here every such constant is a
field of a dataclass parsed from config.json; no size stands anywhere else in the code.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any


class ConfigError(ValueError):
    """A config.json key is missing, of the wrong type, or asks for something unsupported."""


def _require(d: dict, key: str, kind):
    if key not in d:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return _typed(d, key, kind)


def _typed(d: dict, key: str, kind):
    value = d[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if kind is int and isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json: key '{key}' must be {kind.__name__}, got {value!r}")
    return value


def _optional(d: dict, key: str, kind, default):
    if key not in d or d[key] is None:
        return default
    return _typed(d, key, kind)


@dataclass(frozen=True)
class Qwen3Config:
    """config.json of ``Qwen3ForCausalLM`` (dense decoder).

    Field names are the checkpoint's own keys.  ``head_dim`` is explicit and need not equal
    ``hidden_size // num_attention_heads`` (the reference derives head counts from the
    projection widths, ampere_kv/runner.py:69).
    """

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    layer_types: tuple[str, ...] | None = None
    eos_token_id: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = ("Qwen3ForCausalLM",)

    ARCHITECTURE = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen3Config":
        heads = _require(d, "num_attention_heads", int)
        hidden = _require(d, "hidden_size", int)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: 'num_attention_heads' and 'hidden_size' must be positive")
        eos = d.get("eos_token_id")
        if eos is None:
            eos = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos = tuple(eos)
        else:
            raise ConfigError(f"config.json: key 'eos_token_id' must be an int or a list of ints, got {eos!r}")
        layer_types = d.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, (list, tuple)) or not all(isinstance(t, str) for t in layer_types):
                raise ConfigError("config.json: key 'layer_types' must be a list of strings")
            layer_types = tuple(layer_types)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"
        arch = d.get("architectures") or (cls.ARCHITECTURE,)
        cfg = cls(
            vocab_size=_require(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=_require(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_optional(d, "num_key_value_heads", int, heads),
            head_dim=_optional(d, "head_dim", int, hidden // heads),
            intermediate_size=_require(d, "intermediate_size", int),
            rope_theta=_optional(d, "rope_theta", float, 10000.0),
            rms_norm_eps=_optional(d, "rms_norm_eps", float, 1e-6),
            max_position_embeddings=_optional(d, "max_position_embeddings", int, 32768),
            tie_word_embeddings=_optional(d, "tie_word_embeddings", bool, False),
            hidden_act=_optional(d, "hidden_act", str, "silu"),
            attention_bias=_optional(d, "attention_bias", bool, False),
            use_sliding_window=_optional(d, "use_sliding_window", bool, False),
            sliding_window=_optional(d, "sliding_window", int, None),
            max_window_layers=_optional(d, "max_window_layers", int, None),
            layer_types=layer_types,
            eos_token_id=eos,
            torch_dtype=str(dtype),
            architectures=tuple(arch),
        )
        cfg.validate(d)
        return cfg

    def validate(self, raw: dict | None = None) -> None:
        for name in ("vocab_size", "num_hidden_layers", "num_key_value_heads", "head_dim", "intermediate_size",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: key '{name}' must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: 'num_attention_heads' ({self.num_attention_heads}) must be a multiple of "
                f"'num_key_value_heads' ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' must be even for rotate-half RoPE, got {self.head_dim}")
        if self.hidden_act != "silu":
            # the reference refuses anything but SiLU (ampere_kv/runner.py:39-40)
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', got {self.hidden_act!r}")
        if self.rope_theta <= 0 or self.rms_norm_eps <= 0:
            raise ConfigError("config.json: 'rope_theta' and 'rms_norm_eps' must be positive")
        if raw is not None and raw.get("rope_scaling") not in (None, {}):
            scaling = raw["rope_scaling"]
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                # the reference assumes rope_scaling is empty (ampere_kv/runner.py:83)
                raise ConfigError(f"config.json: 'rope_scaling' {kind!r} is not supported (only none/default)")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("config.json: 'use_sliding_window' is true but 'sliding_window' is not a positive int")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"config.json: 'layer_types' has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            bad = sorted(set(self.layer_types) - {"full_attention", "sliding_attention"})
            if bad:
                raise ConfigError(f"config.json: 'layer_types' holds unknown kinds {bad}")

    def window_of_layer(self, index: int) -> int | None:
        """Number of keys (the query's own included) layer ``index`` attends to, or None for all."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        if self.layer_types is not None:
            slides = self.layer_types[index] == "sliding_attention"
        else:
            first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
            slides = index >= first
        return self.sliding_window if slides else None

    def to_dict(self) -> dict[str, Any]:
        out = {}
        for f in fields(self):
            value = getattr(self, f.name)
            if isinstance(value, tuple):
                value = list(value)
            out[f.name] = value
        if len(out["eos_token_id"]) == 0:
            out["eos_token_id"] = None
        elif len(out["eos_token_id"]) == 1:
            out["eos_token_id"] = out["eos_token_id"][0]
        out["model_type"] = "qwen3"
        return out


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as handle:
        try:
            raw = json.load(handle)
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    # The reference stops on ``model.generation_config.eos_token_id`` (ampere_kv/runner.py:331): the ids of
    # generation_config.json where that file carries them (a published checkpoint lists more ids there than in
    # config.json), else config.json's own.
    gen_path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen_path):
        with open(gen_path, "r", encoding="utf-8") as handle:
            try:
                gen = json.load(handle)
            except json.JSONDecodeError as exc:
                raise ConfigError(f"{gen_path}: not valid JSON ({exc})") from exc
        if isinstance(gen, dict) and gen.get("eos_token_id") is not None:
            raw["eos_token_id"] = gen["eos_token_id"]
    return raw
