"""Typed configuration of the Qwen2 decoder, read from its own ``config.json`` keys.

Counterpart of the reference's ``struct Config`` / ``config_parse`` (src/config.h:13-27,
src/config.c:50-132) and of the gate its converter applies to ``config.json``
(scripts/hf/qwen2.ts:90-106). Like the reference, a missing key or a value out of range
is an error whose message names the key; unlike its converter this configuration also
accepts an untied head, a ``head_dim`` that is not ``hidden_size / heads`` (the runtime
supports both: src/config.c:97-98, src/modelfile.c:25-34) and the sliding window
(``sliding_window`` of src/config.c:107, applied as in src/model.c:465-472).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Any, Dict, Mapping, Optional, Tuple

from .registry import register_architecture
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, require_keys

ARCHITECTURE = "Qwen2ForCausalLM"

_REQUIRED = (
    "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
    "num_key_value_heads", "vocab_size", "max_position_embeddings", "rms_norm_eps",
    "rope_theta", "hidden_act", "tie_word_embeddings",
)


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
    return value


def _finite(raw: Mapping[str, Any], key: str) -> float:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ConfigError(f"config.json: {key} must be a finite number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    eos_token_ids: Tuple[int, ...] = ()

    # ---- parsing -------------------------------------------------------------------
    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "Qwen2Config":
        where = "config.json"
        if raw.get("model_type", "qwen2") != "qwen2":
            raise ConfigError(f"{where}: model_type must be \"qwen2\", got {raw.get('model_type')!r}")
        require_keys(raw, _REQUIRED, where)
        if raw["hidden_act"] != "silu":
            raise ConfigError(f"{where}: hidden_act must be \"silu\", got {raw['hidden_act']!r}")
        if raw.get("rope_scaling"):
            raise ConfigError(f"{where}: rope_scaling is not supported for this architecture")
        if not isinstance(raw["tie_word_embeddings"], bool):
            raise ConfigError(f"{where}: tie_word_embeddings must be true or false")
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads")
        if raw.get("head_dim") is not None:
            head_dim = _positive_int(raw, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(f"{where}: hidden_size {hidden} is not a multiple of num_attention_heads {heads}; give head_dim")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: num_key_value_heads {kv_heads} must divide num_attention_heads {heads}")
        if head_dim % 2:
            raise ConfigError(f"{where}: head_dim {head_dim} must be even")
        eps = _finite(raw, "rms_norm_eps")
        if not 0.0 < eps < 1.0:
            raise ConfigError(f"{where}: rms_norm_eps must be in (0, 1), got {eps}")
        theta = _finite(raw, "rope_theta")
        if not theta > 1.0:
            raise ConfigError(f"{where}: rope_theta must be greater than 1, got {theta}")
        layers = _positive_int(raw, "num_hidden_layers")
        use_window = bool(raw.get("use_sliding_window", False))
        window = None
        max_window_layers = layers
        if use_window:
            require_keys(raw, ("sliding_window", "max_window_layers"), where)
            window = _positive_int(raw, "sliding_window")
            mwl = raw["max_window_layers"]
            if isinstance(mwl, bool) or not isinstance(mwl, int) or mwl < 0:
                raise ConfigError(f"{where}: max_window_layers must be a non-negative integer, got {mwl!r}")
            max_window_layers = mwl
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{where}: eos_token_id must be an integer or a list of integers")
        vocab = _positive_int(raw, "vocab_size")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"{where}: eos_token_id {e} is outside the vocabulary of {vocab}")
        return cls(
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=vocab,
            max_position_embeddings=_positive_int(raw, "max_position_embeddings"),
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=raw["tie_word_embeddings"],
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            eos_token_ids=eos_ids,
        )

    def to_json(self) -> Dict[str, Any]:
        """The ``config.json`` that :meth:`from_json` reads back to an equal object."""
        out: Dict[str, Any] = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen2",
            "hidden_act": "silu",
        }
        fields = asdict(self)
        eos = fields.pop("eos_token_ids")
        if len(eos) == 1:
            out["eos_token_id"] = eos[0]
        elif eos:
            out["eos_token_id"] = list(eos)
        if not self.use_sliding_window:
            fields.pop("sliding_window")
            fields.pop("max_window_layers")
        out.update(fields)
        return out

    # ---- what the engine builds from ----------------------------------------------
    def layer_window(self, layer: int) -> Optional[int]:
        """The window of a layer's attention, or None where it sees every key. The first
        ``max_window_layers`` layers see every key; the others see the last
        ``sliding_window`` positions, the current one included (src/model.c:465-472)."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps},
                            {"weight": name})

        position = PartSpec("rope", {"theta": self.rope_theta, "rotary_dim": self.head_dim})
        feed_forward = PartSpec("gated_mlp", {
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "activation": "silu",  # src/vecmath.c:78-81
        }, {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"})
        layers = []
        for number in range(self.num_hidden_layers):
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "heads": self.num_attention_heads,
                "kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qkv_bias": True,  # fixed by the architecture (src/config.c:84)
                "window": self.layer_window(number),
                "scale": 1.0 / math.sqrt(self.head_dim),  # src/kernels.c:1159
                "position": position,
            }, {
                "q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight",
                "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias",
                "v_bias": "self_attn.v_proj.bias",
            })
            layers.append(LayerSpec(
                block="pre_norm",
                mixer=mixer,
                feed_forward=feed_forward,
                mixer_norm=norm("input_layernorm.weight"),
                feed_forward_norm=norm("post_attention_layernorm.weight"),
                weight_prefix=f"model.layers.{number}",
            ))
        return ModelSpec(
            architecture=ARCHITECTURE,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding_name="model.embed_tokens.weight",
            final_norm=norm("weight"),
            final_norm_prefix="model.norm",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            layers=tuple(layers),
            order=tuple(range(self.num_hidden_layers)),
            stop_token_ids=self.eos_token_ids,
        )


register_architecture(ARCHITECTURE, Qwen2Config)
