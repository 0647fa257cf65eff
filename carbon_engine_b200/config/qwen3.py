"""Typed configuration of the Qwen3 dense architecture (``Qwen3ForCausalLM``).

Keys, defaults and meanings are those the reference reads (src/config.rs:446-694):
``num_key_value_heads`` defaults to the head count and ``head_dim`` to hidden/heads
(src/config.rs:469-471), ``rope_theta`` may sit at the top level or under ``rope_parameters`` and
defaults to 10000 (src/config.rs:472-478), ``intermediate_size`` defaults to four times the hidden
width (src/config.rs:643), ``rms_norm_eps`` to 1e-6 (src/config.rs:649),
``max_position_embeddings`` to 4096 (src/config.rs:652), ``tie_word_embeddings`` to false
(src/config.rs:653-657), ``hidden_act`` to "silu" (src/config.rs:663-667).  Qwen3 has per-head
q/k norms and no attention bias (src/config.rs:658-662).

``rope_scaling`` (or ``rope_parameters``) of kind "linear", "llama3" or "yarn" is read with the
reference's keys and defaults (src/config.rs:483-519).  Where the reference warns and continues (an
unknown kind, src/config.rs:520-524) this class refuses the config: a wrong position encoding gives
wrong logits silently.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..parts.rope import RopeScaling, yarn_mscale
from .base import ConfigError, ModelConfig, token_id_list

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


def _need_int(d: Dict[str, Any], key: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
    return v


def _opt_int(d: Dict[str, Any], key: str, default: int) -> int:
    if d.get(key) is None:
        return default
    return _need_int(d, key)


def _opt_float(d: Dict[str, Any], key: str) -> Optional[float]:
    v = d.get(key)
    if v is None or isinstance(v, bool) or not isinstance(v, (int, float)):
        return None
    return float(v)


def _rope_scaling(r: Dict[str, Any], d: Dict[str, Any]) -> Optional[RopeScaling]:
    """``rope_scaling`` / ``rope_parameters`` with the reference's keys and defaults (src/config.rs:483-529)."""
    kind = r.get("rope_type", r.get("type"))
    kind = "default" if kind is None else kind
    factor = _opt_float(r, "factor")
    factor = 1.0 if factor is None else factor
    if kind == "default":
        return None
    if factor <= 0.0:
        raise ConfigError(f"config.json: rope scaling factor {factor} must be positive")

    def number(key: str, default: float) -> float:
        v = _opt_float(r, key)
        return default if v is None else v
    if kind == "linear":
        return RopeScaling("linear", factor)
    if kind == "llama3":
        return RopeScaling("llama3", factor, low_freq_factor=number("low_freq_factor", 1.0),
                           high_freq_factor=number("high_freq_factor", 4.0),
                           original_max_position=_opt_int(r, "original_max_position_embeddings", 8192))
    if kind == "yarn":
        ms, ms_all = _opt_float(r, "mscale"), _opt_float(r, "mscale_all_dim")
        attention = _opt_float(r, "attention_factor")
        if attention is None:
            attention = yarn_mscale(factor, ms) / yarn_mscale(factor, ms_all) if ms is not None and ms_all is not None \
                else yarn_mscale(factor, 1.0)
        original = _opt_int(r, "original_max_position_embeddings", _opt_int(d, "max_position_embeddings", 4096))
        return RopeScaling("yarn", factor, original_max_position=original, beta_fast=number("beta_fast", 32.0),
                           beta_slow=number("beta_slow", 1.0), attention_factor=attention)
    raise ConfigError(f"config.json: rope scaling '{kind}' is not supported (default, linear, llama3, yarn)")


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    rope_scaling: Optional[RopeScaling] = None
    layer_types: Tuple[str, ...] = ()
    sliding_window: Optional[int] = None
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        # multimodal wrappers keep the language model under text_config (src/config.rs:448-451)
        d = raw.get("text_config") if isinstance(raw.get("text_config"), dict) and \
            "hidden_size" in raw["text_config"] else raw
        if raw.get("quantization_config") is not None or d.get("quantization_config") is not None:
            raise ConfigError("config.json: quantised checkpoints (quantization_config) are not supported")
        hidden = _need_int(d, "hidden_size")
        heads = _need_int(d, "num_attention_heads")
        kv_heads = _opt_int(d, "num_key_value_heads", heads)
        head_dim = _opt_int(d, "head_dim", hidden // heads)
        layers = _need_int(d, "num_hidden_layers")
        vocab = _need_int(d, "vocab_size")
        inter = _opt_int(d, "intermediate_size", 4 * hidden)
        max_pos = _opt_int(d, "max_position_embeddings", 4096)
        eps = _opt_float(d, "rms_norm_eps")
        eps = 1e-6 if eps is None else eps

        rope_params = d.get("rope_scaling")
        if rope_params is None:
            rope_params = d.get("rope_parameters")
        theta = _opt_float(d, "rope_theta")
        if theta is None and isinstance(rope_params, dict):
            theta = _opt_float(rope_params, "rope_theta")
        theta = 10000.0 if theta is None else theta
        scaling = _rope_scaling(rope_params, d) if isinstance(rope_params, dict) else None
        partial = _opt_float(d, "partial_rotary_factor")
        if partial is not None and partial != 1.0:
            raise ConfigError("config.json: partial_rotary_factor other than 1.0 is not a Qwen3 dense model")

        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (silu only)")
        if d.get("attention_bias"):
            raise ConfigError("config.json: attention_bias=true is not a Qwen3 dense model")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads={heads} is not a multiple of num_key_value_heads={kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim={head_dim} must be even for rotary embedding")
        if eps <= 0.0:
            raise ConfigError(f"config.json: rms_norm_eps={eps} must be positive")
        if theta <= 0.0:
            raise ConfigError(f"config.json: rope_theta={theta} must be positive")

        tie = raw.get("tie_word_embeddings", d.get("tie_word_embeddings", False))
        if not isinstance(tie, bool):
            raise ConfigError("config.json: tie_word_embeddings must be true or false")

        # layer_types absent means every layer attends to all keys (src/config.rs:606)
        lt = d.get("layer_types")
        window = d.get("sliding_window")
        if lt is None:
            layer_types = tuple([FULL_ATTENTION] * layers)
        else:
            if not isinstance(lt, list) or len(lt) != layers:
                raise ConfigError(f"config.json: layer_types must list {layers} entries")
            for t in lt:
                if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                    raise ConfigError(f"config.json: unknown layer type '{t}'")
            layer_types = tuple(lt)
        if SLIDING_ATTENTION in layer_types:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError("config.json: sliding_attention layers need a positive sliding_window")
        else:
            window = None

        eos = token_id_list(d.get("eos_token_id"))
        for t in raw.get("_generation_eos_token_ids", []):
            if t not in eos:
                eos.append(t)
        bos = d.get("bos_token_id")
        archs = raw.get("architectures") or ["Qwen3ForCausalLM"]
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        return cls(
            architecture=str(archs[0]), vocab_size=vocab, max_position_embeddings=max_pos,
            eos_token_ids=tuple(eos), hidden_size=hidden, intermediate_size=inter,
            num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
            head_dim=head_dim, rms_norm_eps=eps, rope_theta=theta, rope_scaling=scaling, tie_word_embeddings=tie,
            hidden_act=act, layer_types=layer_types, sliding_window=window,
            bos_token_id=bos if isinstance(bos, int) and not isinstance(bos, bool) else None,
            torch_dtype=str(dtype),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            out["rope_scaling"] = {"rope_type": rs.kind, "factor": rs.factor}
            if rs.kind == "llama3":
                out["rope_scaling"].update(low_freq_factor=rs.low_freq_factor, high_freq_factor=rs.high_freq_factor,
                                           original_max_position_embeddings=rs.original_max_position)
            elif rs.kind == "yarn":
                out["rope_scaling"].update(original_max_position_embeddings=rs.original_max_position, beta_fast=rs.beta_fast,
                                           beta_slow=rs.beta_slow, attention_factor=rs.attention_factor)
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if SLIDING_ATTENTION in self.layer_types:
            out["layer_types"] = list(self.layer_types)
            out["sliding_window"] = self.sliding_window
        return out
