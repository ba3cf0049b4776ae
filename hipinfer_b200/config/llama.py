"""`LlamaConfig`: the dense Llama decoder's config.json keys, typed and checked.

Keys and defaults follow what the reference's exporter reads from such a file
(scripts/export.py:203, 230-232: vocab_size, hidden_size, intermediate_size,
num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim or hidden/heads,
max_position_embeddings, rms_norm_eps; rope_theta at 109; rope_scaling printed at 243), plus
the keys the reference never checks but silently relies on (docs/porting-a-model.md "silent"
rows): `hidden_act` must be silu and there are no biases.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


@dataclass(frozen=True)
class Llama3RopeScaling:
    """rope_scaling of rope_type "llama3": per-frequency rescaling by wavelength."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self):
        return dict(rope_type="llama3", factor=self.factor, low_freq_factor=self.low_freq_factor,
                    high_freq_factor=self.high_freq_factor,
                    original_max_position_embeddings=self.original_max_position_embeddings)


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
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
    rope_scaling: Optional[Llama3RopeScaling]
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        heads = take(d, "num_attention_heads", int, positive=True)
        hidden = take(d, "hidden_size", int, positive=True)
        kv = take(d, "num_key_value_heads", int, heads, positive=True)
        head_dim = take(d, "head_dim", int, None, positive=True)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads "
                                  f"{heads} and there is no head_dim")
            head_dim = hidden // heads
        if heads % kv:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even (rotary pairs)")
        act = take(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r}: this architecture's feed-forward is SwiGLU (silu)")
        for key in ("attention_bias", "mlp_bias"):
            if take(d, key, bool, False):
                raise ConfigError(f"config.json: {key} is true: this architecture has no biases")
        theta = take(d, "rope_theta", float, None, positive=True)
        scaling_d = d.get("rope_scaling")
        if theta is None and isinstance(d.get("rope_parameters"), dict):
            # newer files keep theta and the scaling keys together under rope_parameters
            theta = take(d["rope_parameters"], "rope_theta", float, None, positive=True)
            if scaling_d is None and d["rope_parameters"].get("rope_type", "default") != "default":
                scaling_d = d["rope_parameters"]
        if theta is None:
            theta = 10000.0
        scaling = None
        if scaling_d is not None:
            if not isinstance(scaling_d, dict):
                raise ConfigError("config.json: rope_scaling must be an object or null")
            kind = scaling_d.get("rope_type", scaling_d.get("type"))
            if kind in (None, "default"):
                scaling = None
            elif kind == "llama3":
                scaling = Llama3RopeScaling(
                    factor=take(scaling_d, "factor", float, positive=True),
                    low_freq_factor=take(scaling_d, "low_freq_factor", float, positive=True),
                    high_freq_factor=take(scaling_d, "high_freq_factor", float, positive=True),
                    original_max_position_embeddings=take(scaling_d, "original_max_position_embeddings", int,
                                                          positive=True))
                if scaling.high_freq_factor <= scaling.low_freq_factor:
                    raise ConfigError("config.json: rope_scaling.high_freq_factor must exceed low_freq_factor")
            else:
                raise ConfigError(f"config.json: rope_scaling.rope_type {kind!r} is not supported "
                                  f"(supported: 'default', 'llama3')")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: eos_token_id must be an int or a list of ints, got {eos!r}")
        dt = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dt, str):
            raise ConfigError(f"config.json: torch_dtype must be a string, got {dt!r}")
        return cls(
            architecture=d["architectures"][0],
            vocab_size=take(d, "vocab_size", int, positive=True),
            hidden_size=hidden,
            intermediate_size=take(d, "intermediate_size", int, positive=True),
            num_hidden_layers=take(d, "num_hidden_layers", int, positive=True),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            max_position_embeddings=take(d, "max_position_embeddings", int, positive=True),
            rms_norm_eps=take(d, "rms_norm_eps", float, 1e-6, positive=True),
            rope_theta=theta,
            rope_scaling=scaling,
            tie_word_embeddings=take(d, "tie_word_embeddings", bool, False),
            hidden_act=act,
            torch_dtype=dt,
            bos_token_id=take(d, "bos_token_id", int, None),
            eos_token_ids=eos_ids,
        )

    def to_dict(self) -> Dict[str, Any]:
        d = dict(
            architectures=[self.architecture], model_type="llama", vocab_size=self.vocab_size,
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            num_hidden_layers=self.num_hidden_layers, num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
            max_position_embeddings=self.max_position_embeddings, rms_norm_eps=self.rms_norm_eps,
            rope_theta=self.rope_theta, rope_scaling=self.rope_scaling.to_dict() if self.rope_scaling else None,
            tie_word_embeddings=self.tie_word_embeddings, hidden_act=self.hidden_act, attention_bias=False,
            mlp_bias=False, torch_dtype=self.torch_dtype, bos_token_id=self.bos_token_id,
            eos_token_id=list(self.eos_token_ids) if self.eos_token_ids else None)
        return d
