"""Qwen3 dense decoder (``Qwen3ForCausalLM``) as a configuration and a list of parts.

Keys, defaults and checks follow thanhauco/rust-inference's
src/models/config.rs:19-111; tensor names follow src/models/qwen3.rs:157-188.
The model itself is not written here: ``to_spec`` says which parts make a
layer and the generic model in ``engine/model.py`` assembles them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RopeSpec, ScheduleEntry,
                            SwiGLUSpec)

_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads")


def _as_int(d, key):
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {key} must be a non-negative integer, got {v!r}")
    return v


@register_architecture("Qwen3ForCausalLM", "qwen3")
@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int                               # default hidden_size / heads (config.rs:75-77)
    max_position_embeddings: int = 40960        # config.rs:58-60
    rms_norm_eps: float = 1e-6                  # config.rs:61-63
    rope_theta: float = 1_000_000.0             # config.rs:64-66
    tie_word_embeddings: bool = False           # config.rs:35-36
    rope_scaling: Optional[dict] = None         # only null / "default" (config.rs:104-109)
    eos_token_ids: Tuple[int, ...] = ()         # stop ids; int or list in config.json
    extra: Tuple[Tuple[str, object], ...] = field(default=(), compare=False)

    # ---- config.json <-> object -------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks {', '.join(missing)}")
        heads = _as_int(d, "num_attention_heads")
        hd = d.get("head_dim")
        if hd is None:
            if heads == 0:
                raise ConfigError("attention heads must be non-zero")
            hd = _as_int(d, "hidden_size") // heads
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        # Keys the reference never reads (attention_bias, sliding_window, ...) would
        # change the result if they were active, so they are refused, not ignored.
        if d.get("attention_bias"):
            raise ConfigError("attention_bias=true: this Qwen3 has no bias tensors")
        if d.get("use_sliding_window"):
            raise ConfigError("use_sliding_window=true: this Qwen3 attends to all keys")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {d['hidden_act']!r}: the feed-forward is SiLU-gated")
        if d.get("num_experts"):
            raise ConfigError("num_experts > 0 belongs to Qwen3MoeForCausalLM, which is not built here")
        if d.get("quantization_config"):
            raise ConfigError("quantized checkpoints are not supported")
        known = set(_REQUIRED) | {"head_dim", "max_position_embeddings", "rms_norm_eps", "rope_theta",
                                  "tie_word_embeddings", "rope_scaling", "eos_token_id"}
        extra = tuple(sorted((k, _freeze(v)) for k, v in d.items() if k not in known))
        return cls(
            vocab_size=_as_int(d, "vocab_size"), hidden_size=_as_int(d, "hidden_size"),
            intermediate_size=_as_int(d, "intermediate_size"),
            num_hidden_layers=_as_int(d, "num_hidden_layers"), num_attention_heads=heads,
            num_key_value_heads=_as_int(d, "num_key_value_heads"), head_dim=int(hd),
            max_position_embeddings=int(d.get("max_position_embeddings", 40960)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(d.get("rope_theta", 1_000_000.0)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            rope_scaling=d.get("rope_scaling"), eos_token_ids=eos_ids, extra=extra)

    def to_dict(self) -> dict:
        d = {
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta, "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.rope_scaling is not None:
            d["rope_scaling"] = self.rope_scaling
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    # ---- checks (config.rs:87-111) ---------------------------------------------------
    def validate(self) -> None:
        if self.num_attention_heads == 0 or self.num_key_value_heads == 0:
            raise ConfigError("attention heads must be non-zero")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{self.num_attention_heads} attention heads not divisible by "
                              f"{self.num_key_value_heads} kv heads")
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary embeddings")
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "max_position_embeddings"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"{k} must be positive")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            kind = rs.get("rope_type", rs.get("type")) if isinstance(rs, dict) else rs
            if kind not in (None, "default"):
                raise ConfigError(f"rope_scaling {rs} is not supported")

    # ---- the model as parts --------------------------------------------------------
    def to_spec(self) -> ModelSpec:
        D, eps = self.hidden_size, self.rms_norm_eps
        attn = AttentionSpec(
            hidden_size=D, num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            position=RopeSpec(head_dim=self.head_dim, theta=self.rope_theta),
            qk_norm=RMSNormSpec(size=self.head_dim, eps=eps))
        ffn = SwiGLUSpec(hidden_size=D, intermediate_size=self.intermediate_size)
        norm = RMSNormSpec(size=D, eps=eps)
        layers = tuple(
            LayerSpec(mixer=attn, ffn=ffn, mixer_norm=norm, ffn_norm=norm, names=(
                ("mixer", f"model.layers.{i}.self_attn."), ("ffn", f"model.layers.{i}.mlp."),
                ("mixer_norm", f"model.layers.{i}.input_layernorm."),
                ("ffn_norm", f"model.layers.{i}.post_attention_layernorm.")))
            for i in range(self.num_hidden_layers))
        schedule = tuple(ScheduleEntry(layer=i, cache=i) for i in range(self.num_hidden_layers))
        return ModelSpec(
            architecture="Qwen3ForCausalLM", vocab_size=self.vocab_size, hidden_size=D, layers=layers,
            schedule=schedule, final_norm=norm, tie_embeddings=self.tie_word_embeddings,
            max_positions=self.max_position_embeddings, stop_ids=self.eos_token_ids)


def _freeze(v):
    if isinstance(v, list):
        return tuple(_freeze(x) for x in v)
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    return v
