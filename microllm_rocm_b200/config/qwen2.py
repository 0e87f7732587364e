"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

Every size and constant of the model comes from here; nothing in the engine carries a
literal model size.  Keys and their meaning follow the reference's parser
(src/model/huggingface.cpp:142-182) and validation (src/model/config.cpp:27-44), with
three deliberate differences:

* the reference requires every key it reads, including ones it never uses
  (huggingface.cpp:76-102 throws on a missing member); optional keys default here;
* the reference rejects `use_sliding_window=true` (huggingface.cpp:159-161); here a layer
  `l` attends over a window of `sliding_window` keys iff `use_sliding_window` and
  `l >= max_window_layers`;
* `head_dim` may be given; the reference always derives it as hidden/heads
  (config.cpp:46-51).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict, fields
from typing import Any, Dict, Optional

ARCHITECTURE = "Qwen2ForCausalLM"


class ConfigError(ValueError):
    pass


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    max_position_embeddings: int
    rope_theta: float = 10000.0          # reference struct default (config.h:19)
    rms_norm_eps: float = 1e-5           # reference struct default (config.h:24)
    tie_word_embeddings: bool = False
    head_dim: Optional[int] = None       # None: hidden_size // num_attention_heads
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    architectures: tuple = (ARCHITECTURE,)
    model_type: str = "qwen2"

    # ---- derived -----------------------------------------------------------------
    @property
    def head_size(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_size // self.num_attention_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """Number of keys (itself included) that layer `layer` may see, or None for all."""
        if self.use_sliding_window and self.sliding_window is not None and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return None

    def parameter_count(self) -> int:
        """Same count as the reference's ModelConfig::parameter_count (config.cpp:58-78),
        extended by the three projection biases."""
        h, d = self.hidden_size, self.head_size
        q, kv = self.num_attention_heads * d, self.num_key_value_heads * d
        per_layer = (h * q + q) + 2 * (h * kv + kv) + q * h + 3 * h * self.intermediate_size + 2 * h
        total = self.vocab_size * h + self.num_hidden_layers * per_layer + h
        if not self.tie_word_embeddings:
            total += self.vocab_size * h
        return total

    # ---- validation ----------------------------------------------------------------
    def validate(self) -> None:
        ints = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "intermediate_size", "max_position_embeddings")
        for name in ints:
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.model_type != "qwen2":
            raise ConfigError(f"model_type must be 'qwen2', got {self.model_type!r}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act must be 'silu', got {self.hidden_act!r}")
        if self.head_dim is None and self.hidden_size % self.num_attention_heads != 0:
            raise ConfigError("hidden_size must divide into num_attention_heads when head_dim is absent")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_size <= 0 or self.head_size % 2 != 0:
            raise ConfigError("head_dim must be positive and even (rotary pairs)")
        if not (isinstance(self.rope_theta, (int, float)) and math.isfinite(self.rope_theta) and self.rope_theta > 0):
            raise ConfigError("rope_theta must be finite and positive")
        if not (isinstance(self.rms_norm_eps, float) and math.isfinite(self.rms_norm_eps) and self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be finite and positive")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("use_sliding_window needs a positive sliding_window")
            if self.max_window_layers < 0:
                raise ConfigError("max_window_layers must be non-negative")

    # ---- (de)serialisation -----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen2Config":
        raw = dict(raw)
        required = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "intermediate_size", "max_position_embeddings")
        missing = [k for k in required if k not in raw]
        if missing:
            raise ConfigError("config.json is missing " + ", ".join(missing))
        if raw.get("use_mrope", False):
            raise ConfigError("use_mrope=true is not a Qwen2 dense decoder")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported (the reference never reads it)")
        raw.setdefault("num_key_value_heads", raw["num_attention_heads"])
        known = {f.name for f in fields(cls)}
        kwargs = {k: v for k, v in raw.items() if k in known}
        if "architectures" in kwargs:
            kwargs["architectures"] = tuple(kwargs["architectures"])
        for k in ("rope_theta", "rms_norm_eps"):
            if k in kwargs and isinstance(kwargs[k], int) and not isinstance(kwargs[k], bool):
                kwargs[k] = float(kwargs[k])
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen2Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
        if not text or len(text) > 1 << 20:       # same bound as huggingface.cpp:148
            raise ConfigError("config.json size is invalid")
        return cls.from_dict(json.loads(text))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["use_mrope"] = False                    # the reference insists on the key
        if d["head_dim"] is None:
            del d["head_dim"]
        if d["sliding_window"] is None:
            del d["sliding_window"]
        for k in ("bos_token_id", "eos_token_id"):
            if d[k] is None:
                del d[k]
        return d

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=1)


# Named presets: the two tiny test shapes and the three benchmark shapes.
PRESETS: Dict[str, Dict[str, Any]] = {
    "tiny-a": dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=1, intermediate_size=176, max_position_embeddings=128,
                   rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                   use_sliding_window=False, torch_dtype="float32"),
    "tiny-b": dict(vocab_size=384, hidden_size=192, num_hidden_layers=3, num_attention_heads=6,
                   num_key_value_heads=2, intermediate_size=512, max_position_embeddings=256,
                   rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
                   use_sliding_window=True, sliding_window=32, max_window_layers=1,
                   torch_dtype="float32"),
    "qwen2.5-1.5b": dict(vocab_size=151936, hidden_size=1536, num_hidden_layers=28,
                         num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960,
                         max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True),
    "qwen2.5-7b": dict(vocab_size=152064, hidden_size=3584, num_hidden_layers=28,
                       num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
                       max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=False),
    "qwen2.5-14b": dict(vocab_size=152064, hidden_size=5120, num_hidden_layers=48,
                        num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824,
                        max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                        tie_word_embeddings=False),
}


def preset(name: str, **overrides) -> Qwen2Config:
    if name not in PRESETS:
        raise ConfigError(f"unknown preset {name!r}; known: {', '.join(sorted(PRESETS))}")
    raw = dict(PRESETS[name])
    raw.update(overrides)
    return Qwen2Config.from_dict(raw)
