"""Typed configuration of the Llama architecture, read from a Hugging Face ``config.json``.

Keys, defaults and the merge of ``generation_config.json`` follow the reference's
``ModelConfig`` (src/llmserve/config.py:35-79). Two keys that the reference silently ignores are
checked here because a value other than the default would change the math: ``hidden_act`` and
``mlp_bias``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

_ROPE_TYPES = ("default", "linear", "llama3")


class ConfigError(ValueError):
    """A config.json that this engine cannot run."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary tables (src/llmserve/models/layers.py:24-58)."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    @classmethod
    def from_dict(cls, d: dict[str, Any] | None) -> RopeScaling:
        if not d:
            return cls()
        kind = d.get("rope_type", d.get("type")) or "default"
        if kind not in _ROPE_TYPES:
            raise ConfigError(f"rope scaling {kind!r} is not supported; supported: {_ROPE_TYPES}")
        if kind == "default":
            return cls()
        if "factor" not in d:
            raise ConfigError(f"rope scaling {kind!r} needs 'factor'")
        if kind == "llama3" and "original_max_position_embeddings" not in d:
            raise ConfigError("rope scaling 'llama3' needs 'original_max_position_embeddings'")
        return cls(
            rope_type=kind,
            factor=float(d["factor"]),
            low_freq_factor=float(d.get("low_freq_factor", 1.0)),
            high_freq_factor=float(d.get("high_freq_factor", 4.0)),
            original_max_position_embeddings=int(d.get("original_max_position_embeddings", 0)),
        )


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool = False
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    bos_token_id: int | None = None
    eos_token_ids: tuple[int, ...] = ()
    model_type: str = "llama"

    architecture = "LlamaForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> LlamaConfig:
        required = (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
        )
        absent = [k for k in required if k not in d]
        if absent:
            raise ConfigError(f"config.json lacks required keys: {absent}")
        if d.get("model_type", "llama") != "llama":
            raise ConfigError(f"model_type {d.get('model_type')!r} is not 'llama'")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r}: the Llama feed-forward here is SiLU-gated only")
        if d.get("mlp_bias", False):
            raise ConfigError("mlp_bias=true is not supported (the feed-forward has no biases)")
        n_heads = int(d["num_attention_heads"])
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(eos))
        # transformers >= 5 nests the rotary settings in "rope_parameters"
        rope_params = d.get("rope_parameters") or {}
        theta = rope_params.get("rope_theta", d.get("rope_theta", 10000.0))
        scaling = d.get("rope_scaling")
        if scaling is None and rope_params.get("rope_type", "default") != "default":
            scaling = rope_params
        cfg = cls(
            vocab_size=int(d["vocab_size"]),
            hidden_size=int(d["hidden_size"]),
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=n_heads,
            num_key_value_heads=int(d.get("num_key_value_heads", n_heads)),
            head_dim=int(d.get("head_dim") or int(d["hidden_size"]) // n_heads),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(theta),
            max_position_embeddings=int(d.get("max_position_embeddings", 4096)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            rope_scaling=RopeScaling.from_dict(scaling),
            bos_token_id=d.get("bos_token_id"),
            eos_token_ids=eos_ids,
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_pretrained(cls, path: str | Path) -> LlamaConfig:
        path = Path(path)
        cfg = cls.from_dict(json.loads((path / "config.json").read_text()))
        gen = path / "generation_config.json"
        if gen.exists():
            g = json.loads(gen.read_text()).get("eos_token_id")
            extra = () if g is None else ((int(g),) if isinstance(g, int) else tuple(g))
            merged = tuple(dict.fromkeys(cfg.eos_token_ids + extra))
            cfg = cls(**{**cfg.__dict__, "eos_token_ids": merged})
        return cfg

    def validate(self) -> None:
        pos = {
            k: getattr(self, k)
            for k in (
                "vocab_size",
                "hidden_size",
                "intermediate_size",
                "num_hidden_layers",
                "num_attention_heads",
                "num_key_value_heads",
                "head_dim",
                "max_position_embeddings",
            )
        }
        bad = {k: v for k, v in pos.items() if v < 1}
        if bad:
            raise ConfigError(f"sizes must be positive: {bad}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary positions")
        if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` this configuration is read back from."""
        d: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": False,
        }
        if self.rope_scaling.rope_type != "default":
            d["rope_scaling"] = dict(self.rope_scaling.__dict__)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            ids = list(self.eos_token_ids)
            d["eos_token_id"] = ids[0] if len(ids) == 1 else ids
        return d

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def kv_bytes_per_token(self, dtype_bytes: int) -> int:
        """Bytes of K and V that one token holds over all layers (src/llmserve/config.py:81-83)."""
        return 2 * self.num_hidden_layers * self.kv_size * dtype_bytes

    def num_parameters(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = h * (self.q_size + 2 * self.kv_size) + self.q_size * h + 3 * h * i + 2 * h
        if self.attention_bias:
            per_layer += self.q_size + 2 * self.kv_size + h
        head = 0 if self.tie_word_embeddings else v * h
        return v * h + self.num_hidden_layers * per_layer + h + head
