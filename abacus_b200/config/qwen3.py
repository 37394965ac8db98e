"""Typed configuration of the Qwen3 dense decoder, read from config.json.

The keys and their defaults are the ones tools/export.py:76-88 reads. abacus
freezes them into its model file header (src/abacus.h:7-17); here they stay a
typed object. Keys that a Qwen3 config.json carries and abacus never reads
(attention_bias, hidden_act, rope_scaling, the sliding-window keys) are
checked, so that a checkpoint that needs them is refused or honoured, never
silently run wrong.
"""
import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .registry import ConfigError
from .specs import AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, NormSpec, RotarySpec, ScheduleEntry

_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "vocab_size", "max_position_embeddings", "rms_norm_eps")


def _as_int(raw, key, minimum=1):
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {key} must be an integer >= {minimum}, got {v!r}")
    return v


def _as_float(raw, key, v):
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"config.json: {key} must be a positive number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool = False
    layer_types: Tuple[str, ...] = ()
    sliding_window: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    architecture: str = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        if raw.get("model_type", "qwen3") != "qwen3":  # tools/export.py:77-78
            raise ConfigError(f"config.json: expected model_type qwen3, got {raw.get('model_type')!r}")
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        hidden = _as_int(raw, "hidden_size")
        heads = _as_int(raw, "num_attention_heads")
        kv_heads = _as_int(raw, "num_key_value_heads")
        layers = _as_int(raw, "num_hidden_layers")
        head_dim = raw.get("head_dim") or hidden // heads  # tools/export.py:82
        if isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim < 2 or head_dim % 2:
            raise ConfigError(f"config.json: head_dim must be an even integer, got {head_dim!r}")
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_attention_heads {heads} is no multiple of "
                              f"num_key_value_heads {kv_heads}")
        theta = raw.get("rope_theta")
        params = raw.get("rope_parameters") or {}
        if theta is None:  # newer exporters nest it (tools/export.py:83)
            theta = params.get("rope_theta")
        if theta is None:
            raise ConfigError("config.json lacks rope_theta (plain or under rope_parameters)")
        scaling = raw.get("rope_scaling")
        rope_type = (scaling or {}).get("rope_type", (scaling or {}).get("type")) or params.get("rope_type", "default")
        if rope_type not in ("default", None):
            raise ConfigError(f"config.json: rope scaling {rope_type!r} is not built (only plain rotary)")
        if raw.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is not built (abacus has no biases)")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"config.json: hidden_act {raw['hidden_act']!r} is not built (only silu)")

        window = raw.get("sliding_window")
        types = raw.get("layer_types")
        if types is None:
            # older exporters give use_sliding_window / max_window_layers instead of a list
            first_windowed = raw.get("max_window_layers", layers) if raw.get("use_sliding_window", False) else layers
            types = ["sliding_attention" if (window and l >= first_windowed) else "full_attention"
                     for l in range(layers)]
        if len(types) != layers:
            raise ConfigError(f"config.json: layer_types has {len(types)} entries for {layers} layers")
        for t in types:
            if t not in ("full_attention", "sliding_attention"):
                raise ConfigError(f"config.json: layer type {t!r} is not built")
        if "sliding_attention" in types:
            if isinstance(window, bool) or not isinstance(window, int) or window < 1:
                raise ConfigError(f"config.json: sliding_attention layers need sliding_window >= 1, got {window!r}")
        else:
            window = None

        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        return cls(
            hidden_size=hidden, intermediate_size=_as_int(raw, "intermediate_size"), num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            vocab_size=_as_int(raw, "vocab_size"), max_position_embeddings=_as_int(raw, "max_position_embeddings"),
            rope_theta=_as_float(raw, "rope_theta", theta), rms_norm_eps=_as_float(raw, "rms_norm_eps", raw["rms_norm_eps"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),  # tools/export.py:81
            layer_types=tuple(types), sliding_window=window, eos_token_ids=eos)

    def to_dict(self):
        """A config.json that from_dict reads back to this object."""
        d = {
            "architectures": [self.architecture], "model_type": "qwen3",
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "vocab_size": self.vocab_size, "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings, "layer_types": list(self.layer_types),
            "sliding_window": self.sliding_window, "use_sliding_window": self.sliding_window is not None,
            "attention_bias": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    def to_spec(self):
        """The parts of every layer, in abacus's arrangement (src/model.c:286-313)."""
        rotary = RotarySpec(theta=self.rope_theta, rotary_dim=self.head_dim, pairing="half")  # src/model.c:173-181
        layers = []
        for l in range(self.num_hidden_layers):
            mixer = AttentionSpec(
                hidden=self.hidden_size, n_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim, scale=1.0 / math.sqrt(self.head_dim),  # src/model.c:202
                qk_norm_eps=self.rms_norm_eps,  # src/model.c:251-252: same eps as the layer norms
                position=rotary,
                window=self.sliding_window if self.layer_types[l] == "sliding_attention" else None)
            layers.append(BlockSpec(
                mixer_norm=NormSpec(self.hidden_size, self.rms_norm_eps), mixer=mixer,
                ffn_norm=NormSpec(self.hidden_size, self.rms_norm_eps),
                ffn=GatedMLPSpec(self.hidden_size, self.intermediate_size, "silu"), arrangement="pre_norm"))
        return ModelSpec(
            architecture=self.architecture, hidden=self.hidden_size, vocab=self.vocab_size, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(l) for l in range(self.num_hidden_layers)),
            final_norm=NormSpec(self.hidden_size, self.rms_norm_eps), tied_head=self.tie_word_embeddings,
            max_positions=self.max_position_embeddings, stop_tokens=self.eos_token_ids)
