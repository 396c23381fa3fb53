"""Configuration of the Qwen3 dense decoder, from its ``config.json`` keys.

Keys, defaults and checks follow wick ``src/config.rs:55-133``: required sizes
(``config.rs:69-71,110-115``), ``num_key_value_heads`` defaulting to the head
count (``:72``), a ``head_dim`` that is decoupled from ``hidden_size / heads``
(``:73``), ``rope_theta`` either at top level or inside ``rope_parameters``
(``:79-86``), ``rms_norm_eps`` 1e-6 and ``max_position_embeddings`` 4096 when
absent (``:116-117``), and the two divisibility checks (``:126-131``).

The reference never reads the sliding-window keys and would compute full
attention for a checkpoint that asks for a window; this class refuses such a
configuration instead of producing different numbers than the checkpoint's
authors intended.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import (ConfigError, ModelConfig, need_int, opt_bool, opt_float,
                   opt_int, token_ids)


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    # ---- derived sizes (config.rs:153-159) ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def vocab(self) -> int:
        return self.vocab_size

    @property
    def max_position(self) -> int:
        return self.max_position_embeddings

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return self.eos_token_ids

    def param_count(self, tied: Optional[bool] = None) -> int:
        """Number of parameters (model.rs:240-244)."""
        tied = self.tie_word_embeddings if tied is None else tied
        h, ff = self.hidden_size, self.intermediate_size
        per_layer = h * (2 * self.q_dim + 2 * self.kv_dim) + 3 * h * ff + 2 * h + 2 * self.head_dim
        return self.vocab_size * h * (1 if tied else 2) + self.num_hidden_layers * per_layer + h

    def validate(self) -> None:
        if self.num_attention_heads <= 0 or self.num_key_value_heads <= 0:
            raise ConfigError("config.json: missing num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2 != 0 or self.head_dim <= 0:
            raise ConfigError("head_dim must be even for rotary embeddings")
        for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size",
                  "max_position_embeddings"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: {k} must be positive")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError("config.json: rope_theta must be positive")

    @classmethod
    def from_json(cls, j: Mapping[str, Any], architecture: str = "Qwen3ForCausalLM") -> "Qwen3Config":
        hidden = need_int(j, "hidden_size")
        heads = need_int(j, "num_attention_heads")
        if heads == 0:
            raise ConfigError("config.json: missing num_attention_heads")
        kv_heads = opt_int(j, "num_key_value_heads", heads)
        head_dim = opt_int(j, "head_dim", hidden // heads)
        act = j.get("hidden_act")
        if isinstance(act, str) and act != "silu":
            raise ConfigError(f"unsupported activation {act}")
        rope_params = j.get("rope_parameters")
        if not isinstance(rope_params, dict):
            rope_params = None
        theta = j.get("rope_theta")
        if isinstance(theta, bool) or not isinstance(theta, (int, float)):
            theta = rope_params.get("rope_theta") if rope_params else None
        if isinstance(theta, bool) or not isinstance(theta, (int, float)):
            theta = 10000.0
        scaling = j.get("rope_scaling")
        if not isinstance(scaling, dict):
            scaling = rope_params
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type", "default"))
            if not isinstance(kind, str):
                kind = "default"
            if kind != "default":
                raise ConfigError(f"unsupported rope_scaling type {kind!r}")
        if opt_bool(j, "attention_bias", False):
            raise ConfigError("unsupported attention_bias true: the Qwen3 dense decoder has no projection biases")
        window = j.get("sliding_window")
        if opt_bool(j, "use_sliding_window", False) and window is not None:
            raise ConfigError("unsupported use_sliding_window true: only full attention layers are built")
        lt = j.get("layer_types")
        if isinstance(lt, list):
            bad = sorted({str(x) for x in lt if x != "full_attention"})
            if bad:
                raise ConfigError(f"unsupported layer_types {bad}: only full_attention layers are built")
        bos = j.get("bos_token_id")
        cfg = cls(
            architecture=architecture,
            hidden_size=hidden,
            intermediate_size=need_int(j, "intermediate_size"),
            num_hidden_layers=need_int(j, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=need_int(j, "vocab_size"),
            max_position_embeddings=opt_int(j, "max_position_embeddings", 4096),
            rms_norm_eps=opt_float(j, "rms_norm_eps", 1e-6),
            rope_theta=float(theta),
            tie_word_embeddings=opt_bool(j, "tie_word_embeddings", False),
            bos_token_id=bos if isinstance(bos, int) and not isinstance(bos, bool) else None,
            eos_token_ids=token_ids(j.get("eos_token_id")),
        )
        cfg.validate()
        return cfg

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = {
            "architectures": ["Qwen3ForCausalLM" if self.architecture == "qwen3" else self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.bos_token_id is not None:
            j["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            j["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return j
