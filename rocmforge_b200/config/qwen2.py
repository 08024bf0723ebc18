"""Typed configuration of the Qwen2.5 dense decoder, read from its own config.json keys.

Counterpart of maeddesg/ROCmForge's ``ModelConfig`` (src/config.rs:528-569) and of the
key aliases it accepts (src/loader/metadata.rs:70-143); validation follows
src/config.rs:647-680 (all sizes non-zero, heads divisible by kv heads, head_dim not
tied to hidden/heads) and adds what the kernels need.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import List, Optional

from .errors import InvalidValue, MissingKey


def _req_int(raw, key, minimum=1):
    if key not in raw or raw[key] is None:
        raise MissingKey(key)
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise InvalidValue(key, v, "must be an integer")
    if v < minimum:
        raise InvalidValue(key, v, f"must be >= {minimum}")
    return v


def _opt_int(raw, key, default, minimum=1):
    if raw.get(key) is None:
        return default
    return _req_int(raw, key, minimum)


def _req_float(raw, key, default=None):
    v = raw.get(key, default)
    if v is None:
        raise MissingKey(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise InvalidValue(key, v, "must be a number")
    if not v > 0:
        raise InvalidValue(key, v, "must be positive")
    return float(v)


@dataclass
class Qwen2Config:
    architecture: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    hidden_act: str
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    eos_token_ids: List[int]
    torch_dtype: str

    ARCHITECTURE = "Qwen2ForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        archs = raw.get("architectures") or [cls.ARCHITECTURE]
        nh = _req_int(raw, "num_attention_heads")
        hidden = _req_int(raw, "hidden_size")
        # src/config.rs:587 — kv heads default to the number of heads
        nkv = _opt_int(raw, "num_key_value_heads", nh)
        # src/loader/metadata.rs:130-143 — explicit head_dim, else hidden / heads
        hd = _opt_int(raw, "head_dim", None)
        if hd is None:
            if hidden % nh:
                raise InvalidValue("hidden_size", hidden,
                                   f"not divisible by num_attention_heads={nh} and no head_dim given")
            hd = hidden // nh
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = [eos]
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = list(eos)
        else:
            raise InvalidValue("eos_token_id", eos, "must be an integer or a list of integers")
        usw = raw.get("use_sliding_window", False)
        if not isinstance(usw, bool):
            raise InvalidValue("use_sliding_window", usw, "must be true or false")
        tie = raw.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise InvalidValue("tie_word_embeddings", tie, "must be true or false")
        cfg = cls(
            architecture=archs[0],
            num_hidden_layers=_req_int(raw, "num_hidden_layers"),
            hidden_size=hidden,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=hd,
            intermediate_size=_req_int(raw, "intermediate_size"),
            vocab_size=_req_int(raw, "vocab_size"),
            # src/loader/metadata.rs:98-101 with the reference's default of 2048
            max_position_embeddings=_opt_int(raw, "max_position_embeddings", 2048),
            # src/config.rs:422-423 — qwen2 defaults
            rms_norm_eps=_req_float(raw, "rms_norm_eps", 1e-6),
            rope_theta=_req_float(raw, "rope_theta", 1e6),
            tie_word_embeddings=tie,
            hidden_act=raw.get("hidden_act", "silu"),
            use_sliding_window=usw,
            sliding_window=_opt_int(raw, "sliding_window", None),
            max_window_layers=_opt_int(raw, "max_window_layers", 0, minimum=0),
            eos_token_ids=eos_ids,
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )
        if raw.get("rope_scaling") is not None:
            raise InvalidValue("rope_scaling", raw["rope_scaling"],
                               "scaled rotary frequencies are not part of this architecture")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            # src/config.rs:664-669
            raise InvalidValue("num_key_value_heads", self.num_key_value_heads,
                               f"num_attention_heads={self.num_attention_heads} is not a multiple of it")
        if self.head_dim % 2:
            raise InvalidValue("head_dim", self.head_dim, "rotation pairs need an even head_dim")
        if self.hidden_act != "silu":
            # the reference fixes SiLU in code (hip_kernels/elementwise.hip:80)
            raise InvalidValue("hidden_act", self.hidden_act, "only 'silu' is defined for this architecture")
        if self.use_sliding_window and self.sliding_window is None:
            raise InvalidValue("sliding_window", None, "use_sliding_window is true but no window is given")
        for tid in self.eos_token_ids:
            if not 0 <= tid < self.vocab_size:
                raise InvalidValue("eos_token_id", tid, f"outside the vocabulary of {self.vocab_size}")

    def window_of_layer(self, layer: int) -> Optional[int]:
        """Number of keys (the query's own included) a layer attends to, None = all."""
        if self.use_sliding_window and self.sliding_window is not None \
                and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_dict(self) -> dict:
        """The config.json that reads back to this configuration."""
        d = asdict(self)
        d.pop("architecture")
        eos = d.pop("eos_token_ids")
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen2"
        if eos:
            d["eos_token_id"] = eos[0] if len(eos) == 1 else eos
        return d
