"""Gemma-2's configuration, read from the keys of its config.json.

The keys and their defaults follow what the reference's exporter reads from the
model's config object (model/export_gemma.py:40-46): layer count, widths, head
counts, ``head_dim``, ``rms_norm_eps``, ``rope_theta`` (10000.0 if absent),
``attn_logit_softcapping`` and ``final_logit_softcapping`` (absent, null or 0
mean "off"), ``query_pre_attn_scalar`` (``head_dim`` if absent).  The reference
asserts ``query_pre_attn_scalar == head_dim`` and that every width is a multiple
of 256 (model/export_gemma.py:47-49); neither restriction exists here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, _get, _id_list

_ACTIVATIONS = ("gelu_pytorch_tanh",)
_LAYER_TYPES = ("sliding_attention", "full_attention")


@dataclass(frozen=True)
class Gemma2Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    sliding_window: Optional[int]
    query_pre_attn_scalar: float
    attn_logit_softcapping: Optional[float]
    final_logit_softcapping: Optional[float]
    hidden_activation: str
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_types: Tuple[str, ...]
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Tuple[int, ...] = ()

    # -- derived ------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def attention_scale(self) -> float:
        return float(self.query_pre_attn_scalar) ** -0.5

    def is_sliding(self, layer: int) -> bool:
        return self.layer_types[layer] == "sliding_attention"

    # -- reading ------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Gemma2Config":
        L = _get(d, "num_hidden_layers", int)
        H = _get(d, "hidden_size", int)
        nh = _get(d, "num_attention_heads", int)
        nkv = _get(d, "num_key_value_heads", int, nh)
        hd = _get(d, "head_dim", int)
        I = _get(d, "intermediate_size", int)
        V = _get(d, "vocab_size", int)
        eps = _get(d, "rms_norm_eps", float, 1e-6)
        theta = _get(d, "rope_theta", float, 10000.0)
        window = _get(d, "sliding_window", int, None, nullable=True)
        qpas = _get(d, "query_pre_attn_scalar", float, float(hd))
        attn_cap = _get(d, "attn_logit_softcapping", float, None, nullable=True)
        final_cap = _get(d, "final_logit_softcapping", float, None, nullable=True)
        # both spellings occur in Gemma-2 config files
        act = _get(d, "hidden_activation", str, None, nullable=True)
        if act is None:
            act = _get(d, "hidden_act", str, "gelu_pytorch_tanh", nullable=True) or "gelu_pytorch_tanh"
        tie = _get(d, "tie_word_embeddings", bool, True)
        max_pos = _get(d, "max_position_embeddings", int, 8192)

        for key, v in (("num_hidden_layers", L), ("hidden_size", H), ("num_attention_heads", nh),
                       ("num_key_value_heads", nkv), ("head_dim", hd), ("intermediate_size", I),
                       ("vocab_size", V), ("max_position_embeddings", max_pos)):
            if v <= 0:
                raise ConfigError(f"config.json: key '{key}' must be positive, got {v}")
        if nh % nkv != 0:
            raise ConfigError(f"config.json: 'num_attention_heads' ({nh}) must be a multiple of "
                              f"'num_key_value_heads' ({nkv})")
        if hd % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' ({hd}) must be even (rotary pairs)")
        if not (eps > 0):
            raise ConfigError(f"config.json: 'rms_norm_eps' must be positive, got {eps}")
        if not (theta > 0):
            raise ConfigError(f"config.json: 'rope_theta' must be positive, got {theta}")
        if not (qpas > 0):
            raise ConfigError(f"config.json: 'query_pre_attn_scalar' must be positive, got {qpas}")
        if window is not None and window <= 0:
            raise ConfigError(f"config.json: 'sliding_window' must be positive or null, got {window}")
        # 0 means "off", as in the exporter's `or 0.0` (model/export_gemma.py:44-45)
        if attn_cap is not None and attn_cap <= 0:
            attn_cap = None
        if final_cap is not None and final_cap <= 0:
            final_cap = None
        if act not in _ACTIVATIONS:
            raise ConfigError(f"config.json: 'hidden_activation' is '{act}'; this architecture "
                              f"computes {', '.join(_ACTIVATIONS)} only")

        lt = d.get("layer_types")
        if lt is None:
            # Gemma-2's rule: layers with an even index slide, odd ones see everything.
            lt = ["sliding_attention" if (i % 2 == 0) else "full_attention" for i in range(L)]
        if not (isinstance(lt, (list, tuple)) and len(lt) == L and all(x in _LAYER_TYPES for x in lt)):
            raise ConfigError(f"config.json: 'layer_types' must list {L} entries out of {_LAYER_TYPES}")
        if window is None:
            lt = ["full_attention"] * L

        return cls(num_hidden_layers=L, hidden_size=H, num_attention_heads=nh, num_key_value_heads=nkv,
                   head_dim=hd, intermediate_size=I, vocab_size=V, rms_norm_eps=eps, rope_theta=theta,
                   sliding_window=window, query_pre_attn_scalar=qpas, attn_logit_softcapping=attn_cap,
                   final_logit_softcapping=final_cap, hidden_activation=act, tie_word_embeddings=tie,
                   max_position_embeddings=max_pos, layer_types=tuple(lt),
                   eos_token_id=_id_list(d, "eos_token_id"), bos_token_id=_id_list(d, "bos_token_id"))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        def ids(t):
            return None if not t else (t[0] if len(t) == 1 else list(t))
        return {
            "architectures": ["Gemma2ForCausalLM"],
            "model_type": "gemma2",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "sliding_window": self.sliding_window,
            "query_pre_attn_scalar": self.query_pre_attn_scalar,
            "attn_logit_softcapping": self.attn_logit_softcapping,
            "final_logit_softcapping": self.final_logit_softcapping,
            "hidden_activation": self.hidden_activation,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "layer_types": list(self.layer_types),
            "eos_token_id": ids(self.eos_token_id),
            "bos_token_id": ids(self.bos_token_id),
            "torch_dtype": "bfloat16",
        }
