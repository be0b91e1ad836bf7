"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference has no typed model config: it reads attributes off the Hugging Face
config object (src/flexengine/inference/models/qwen2.py:25-45) and rejects what it
does not implement (qwen2.py:26-39).  Here the same keys, defaults and rejections
are a frozen dataclass that is built straight from the JSON file, so that no size
or constant of a model lives anywhere in code.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Mapping


class ConfigError(ValueError):
    """Raised for a config.json that is malformed or asks for something unsupported."""


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder {model_dir!r}")
    with open(path, "r", encoding="utf8") as f:
        data = json.load(f)
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return data


def _require(data: Mapping[str, Any], key: str, kind):
    if key not in data or data[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    value = data[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: {key!r} must be an integer, got {value!r}")
        return int(value)
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: {key!r} must be a number, got {value!r}")
        return float(value)
    return value


@dataclass(frozen=True)
class Qwen2Config:
    """Configuration of a ``Qwen2ForCausalLM`` (Qwen2 / Qwen2.5 dense decoder).

    Keys and defaults follow what the reference reads (qwen2.py:25-45):
    ``head_dim`` defaults to ``hidden_size // num_attention_heads`` (qwen2.py:36),
    ``rope_theta`` to 10000.0 and may come from ``rope_scaling["rope_theta"]`` when
    the scaling type is "default" (qwen2.py:42-45); sliding-window attention and any
    real RoPE scaling are rejected (qwen2.py:28-33); the GQA ratio must be whole
    (qwen2.py:38-39).
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 0
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    eos_token_ids: tuple = ()
    bos_token_id: int | None = None
    torch_dtype: str = "bfloat16"
    model_type: str = "qwen2"
    architectures: tuple = ("Qwen2ForCausalLM",)
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    ARCHITECTURE = "Qwen2ForCausalLM"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen2Config":
        model_type = data.get("model_type")
        if model_type != "qwen2":
            raise ConfigError("Only Qwen2/Qwen2.5 models with model_type=qwen2 are supported "
                              f"(got model_type={model_type!r})")
        if data.get("use_sliding_window", False):
            raise ConfigError("Sliding-window attention is not implemented (use_sliding_window=true)")
        rope_scaling = data.get("rope_scaling")
        rope_type = None
        if isinstance(rope_scaling, dict):
            rope_type = rope_scaling.get("rope_type", rope_scaling.get("type"))
        if rope_scaling and rope_type != "default":
            raise ConfigError(f"RoPE scaling is not implemented (rope_scaling={rope_scaling!r})")
        theta = data.get("rope_theta")
        if theta is None and rope_type == "default":
            theta = rope_scaling.get("rope_theta")
        theta = float(theta) if theta is not None else 10000.0

        hidden = _require(data, "hidden_size", int)
        nq = _require(data, "num_attention_heads", int)
        nkv = data.get("num_key_value_heads")
        nkv = nq if nkv is None else _require(data, "num_key_value_heads", int)
        if nq <= 0 or nkv <= 0:
            raise ConfigError("head counts must be positive")
        if nq % nkv:
            raise ConfigError(f"Invalid GQA head ratio: {nq} query heads over {nkv} key/value heads")
        head_dim = data.get("head_dim")
        if head_dim is None:
            if hidden % nq:
                raise ConfigError("hidden_size is not a multiple of num_attention_heads and head_dim is absent")
            head_dim = hidden // nq
        head_dim = int(head_dim)
        act = data.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not implemented (the SwiGLU feed-forward uses silu)")
        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        known = {f.name for f in fields(cls)} | {"eos_token_id", "rope_scaling", "num_key_value_heads"}
        cfg = cls(
            vocab_size=_require(data, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_require(data, "intermediate_size", int),
            num_hidden_layers=_require(data, "num_hidden_layers", int),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            rms_norm_eps=_require(data, "rms_norm_eps", float),
            rope_theta=theta,
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            max_position_embeddings=int(data.get("max_position_embeddings", 0) or 0),
            hidden_act=act,
            use_sliding_window=False,
            eos_token_ids=eos_ids,
            bos_token_id=(None if data.get("bos_token_id") is None else int(data["bos_token_id"])),
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
            model_type="qwen2",
            architectures=tuple(data.get("architectures") or (cls.ARCHITECTURE,)),
            extra={k: v for k, v in data.items() if k not in known},
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "head_dim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive")
        if self.head_dim % 2:
            raise ConfigError("head_dim must be even for rotary position encoding")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError("rms_norm_eps must be positive")
        if not (self.rope_theta > 0.0):
            raise ConfigError("rope_theta must be positive")

    def to_dict(self) -> dict:
        """The config.json form of this configuration (round-trips through from_dict)."""
        d = asdict(self)
        d.pop("extra")
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        d["architectures"] = list(self.architectures)
        d.update(self.extra)
        return d

    def parameter_count(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        qd, kd = self.num_attention_heads * self.head_dim, self.num_key_value_heads * self.head_dim
        per_layer = (qd + 2 * kd) * h + (qd + 2 * kd) + qd * h + 3 * h * i + 2 * h
        return self.num_hidden_layers * per_layer + v * h * (1 if self.tie_word_embeddings else 2) + h
