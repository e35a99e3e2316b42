"""Typed configuration of the Llama 3 dense decoder, read from config.json.

The reference builds its `Config` from GGUF metadata keys (src/model.rs:16-54,
src/model.rs:138-233: `embedding_length`, `attention.head_count`,
`attention.head_count_kv` defaulting to the head count, `attention.key_length`
defaulting to dim / heads, `rope.freq_base` defaulting to 10000,
`attention.layer_norm_rms_epsilon` defaulting to 1e-5).  Here the same
quantities come from the architecture's own config.json keys; the key
correspondence is the one the reference's converter uses
(scripts/csm-convert.py:49-60).  No size lives in code: everything a layer
needs is a field of this record.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, ClassVar, Mapping, Optional, Tuple

from .errors import ConfigError


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of kind "llama3": per-pair frequency divisors.

    The reference only consumes the result, a table `rope_freqs` of "what the
    plain frequency is divided by" (src/model.rs:30-31, src/model.rs:768); the
    derivation from these four numbers is done by `parts.rope.rotary_inv_freq`.
    """

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


def _need(d: Mapping[str, Any], key: str, arch: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json of {arch}: missing key \"{key}\"")
    return d[key]


def _as_int(name: str, v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: \"{name}\" must be an integer, got {v!r}")
    return int(v)


def _as_float(name: str, v: Any) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: \"{name}\" must be a number, got {v!r}")
    return float(v)


def _token_ids(name: str, v: Any) -> Tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, (list, tuple)):
        return tuple(_as_int(name, t) for t in v)
    return (_as_int(name, v),)


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)
    model_type: ClassVar[str] = "llama"      # what config.json calls this family; written into folders this library makes

    # ---- derived sizes (the reference's kv_dim / q_dim helpers, src/model.rs:255-281)
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def attention_scale(self) -> float:
        """1/sqrt(head_dim), src/model.rs:271."""
        return 1.0 / math.sqrt(self.head_dim)

    def validate(self) -> None:
        pos = {
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
        }
        for k, v in pos.items():
            if v <= 0:
                raise ConfigError(f"config.json: \"{k}\" must be positive, got {v}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")
        rs = self.rope_scaling
        if rs is not None:
            if rs.rope_type != "llama3":
                raise ConfigError(f"config.json: rope_scaling type \"{rs.rope_type}\" is not supported (supported: llama3)")
            if rs.factor <= 0 or rs.high_freq_factor <= rs.low_freq_factor or rs.original_max_position_embeddings <= 0:
                raise ConfigError(
                    "config.json: rope_scaling needs factor > 0, high_freq_factor > low_freq_factor and "
                    "original_max_position_embeddings > 0")
        for t in self.eos_token_ids:
            if not (0 <= t < self.vocab_size):
                raise ConfigError(f"config.json: eos_token_id {t} is outside the vocabulary ({self.vocab_size})")

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures") or []
        arch = archs[0] if archs else "LlamaForCausalLM"
        hidden = _as_int("hidden_size", _need(d, "hidden_size", arch))
        heads = _as_int("num_attention_heads", _need(d, "num_attention_heads", arch))
        kv = d.get("num_key_value_heads")
        kv = heads if kv is None else _as_int("num_key_value_heads", kv)
        hd = d.get("head_dim")
        if hd is None:
            if heads <= 0 or hidden % heads != 0:
                raise ConfigError(f"config.json: hidden_size ({hidden}) is not a multiple of num_attention_heads ({heads}) and head_dim is not given")
            hd = hidden // heads
        else:
            hd = _as_int("head_dim", hd)
        rs_raw = d.get("rope_scaling")
        rs = None
        if rs_raw is not None:
            if not isinstance(rs_raw, Mapping):
                raise ConfigError("config.json: rope_scaling must be an object or null")
            kind = rs_raw.get("rope_type", rs_raw.get("type"))
            if kind in (None, "default"):
                rs = None
            elif kind == "llama3":
                rs = RopeScaling(
                    rope_type="llama3",
                    factor=_as_float("rope_scaling.factor", _need(rs_raw, "factor", arch)),
                    low_freq_factor=_as_float("rope_scaling.low_freq_factor", _need(rs_raw, "low_freq_factor", arch)),
                    high_freq_factor=_as_float("rope_scaling.high_freq_factor", _need(rs_raw, "high_freq_factor", arch)),
                    original_max_position_embeddings=_as_int(
                        "rope_scaling.original_max_position_embeddings",
                        _need(rs_raw, "original_max_position_embeddings", arch)),
                )
            else:
                raise ConfigError(f"config.json: rope_scaling type \"{kind}\" is not supported (supported: llama3)")
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ConfigError("config.json: attention_bias / mlp_bias are not supported (the Llama 3 decoder has no biases)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act \"{act}\" is not supported (supported: silu)")
        known = {
            "architectures", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
            "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings", "rope_theta", "rope_scaling",
            "rms_norm_eps", "tie_word_embeddings", "eos_token_id", "bos_token_id", "torch_dtype", "dtype",
            "attention_bias", "mlp_bias", "hidden_act", "model_type",
        }
        cfg = cls(
            architecture=arch,
            hidden_size=hidden,
            num_hidden_layers=_as_int("num_hidden_layers", _need(d, "num_hidden_layers", arch)),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=hd,
            intermediate_size=_as_int("intermediate_size", _need(d, "intermediate_size", arch)),
            vocab_size=_as_int("vocab_size", _need(d, "vocab_size", arch)),
            max_position_embeddings=_as_int("max_position_embeddings", _need(d, "max_position_embeddings", arch)),
            rope_theta=_as_float("rope_theta", d.get("rope_theta", 10000.0)),
            rope_scaling=rs,
            rms_norm_eps=_as_float("rms_norm_eps", d.get("rms_norm_eps", 1e-5)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=_token_ids("eos_token_id", d.get("eos_token_id")),
            bos_token_id=None if d.get("bos_token_id") is None else _as_int("bos_token_id", d.get("bos_token_id")),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            out["rope_scaling"] = {
                "rope_type": rs.rope_type,
                "factor": rs.factor,
                "low_freq_factor": rs.low_freq_factor,
                "high_freq_factor": rs.high_freq_factor,
                "original_max_position_embeddings": rs.original_max_position_embeddings,
            }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out
