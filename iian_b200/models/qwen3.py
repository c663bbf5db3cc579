"""Qwen3 dense: typed configuration, layer description and tensor names.

Formulas and their order follow the reference's plug-in, src/iian/arch/qwen3.cpp:61-104:
pre-norm RMSNorm, separate Q/K/V projections (biases only if the file has them, :37-47),
RMSNorm over the head axis of Q and K with one weight per projection shared by all heads
(:51-52, :82-87), NEOX rotary positions on the whole head (:66, :106), attention scale
1/sqrt(head_dim) (:72), SiLU-gated parallel feed-forward (:97), optional tied output (:26-27).
The reference reads GGUF keys (src/iian/model_loader.cpp:37-111); the ``config.json`` keys
below carry the same quantities.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


class ConfigError(ValueError):
    pass


def _need(raw: Mapping[str, Any], key: str, kind=int):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: missing required key '{key}'")
    val = raw[key]
    if kind is int:
        if isinstance(val, bool) or not isinstance(val, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {val!r}")
        if val <= 0:
            raise ConfigError(f"config.json: '{key}' must be positive, got {val}")
    return val


def _opt(raw: Mapping[str, Any], key: str, default, kind):
    val = raw.get(key)
    if val is None:
        return default
    if kind is float:
        if isinstance(val, bool) or not isinstance(val, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {val!r}")
        return float(val)
    if kind is int:
        if isinstance(val, bool) or not isinstance(val, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {val!r}")
        return val
    if kind is bool:
        if not isinstance(val, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {val!r}")
        return val
    return val


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    sliding_window: Optional[int] = None        # keys visible to a windowed layer (incl. the query's own)
    layer_types: Tuple[str, ...] = ()            # "full_attention" | "sliding_attention" per layer
    hidden_act: str = "silu"
    eos_token_ids: Tuple[int, ...] = ()          # config.json "eos_token_id": one id or a list

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def window_of_layer(self, i: int) -> Optional[int]:
        return self.sliding_window if self.layer_types[i] == "sliding_attention" else None

    def num_parameters(self) -> int:
        h, f = self.hidden_size, self.intermediate_size
        per_layer = h * (self.q_size + 2 * self.kv_size) + self.q_size * h + 3 * h * f + 2 * h + 2 * self.head_dim
        n = self.num_hidden_layers * per_layer + self.vocab_size * h + h
        if not self.tie_word_embeddings:
            n += self.vocab_size * h
        return n


def qwen3_config_from_dict(raw: Mapping[str, Any]) -> Qwen3Config:
    heads = _need(raw, "num_attention_heads")
    hidden = _need(raw, "hidden_size")
    layers = _need(raw, "num_hidden_layers")
    kv_heads = _opt(raw, "num_key_value_heads", heads, int)        # default = heads (model_loader.cpp:56-58)
    if kv_heads <= 0 or heads % kv_heads != 0:
        raise ConfigError(f"config.json: num_attention_heads ({heads}) must be a multiple of "
                          f"num_key_value_heads ({kv_heads})")
    head_dim = _opt(raw, "head_dim", None, int)
    if head_dim is None:                                             # default hidden/heads; an explicit key wins
        if hidden % heads != 0:
            raise ConfigError(f"config.json: no 'head_dim' and hidden_size ({hidden}) is not a multiple of "
                              f"num_attention_heads ({heads})")
        head_dim = hidden // heads
    if head_dim <= 0 or head_dim % 2 != 0:
        raise ConfigError(f"config.json: 'head_dim' must be positive and even (rotary pairs), got {head_dim}")
    act = raw.get("hidden_act", "silu")
    if act != "silu":
        raise ConfigError(f"config.json: hidden_act '{act}' is not supported by Qwen3 (silu only)")
    scaling = raw.get("rope_scaling")
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
        if kind not in (None, "default"):
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported (Qwen3 passes no frequency "
                              f"factors, src/iian/arch/qwen3.cpp:84)")
    window = _opt(raw, "sliding_window", None, int)
    use_window = _opt(raw, "use_sliding_window", False, bool)
    layer_types = raw.get("layer_types")
    if layer_types is not None:
        if not isinstance(layer_types, list) or len(layer_types) != layers:
            raise ConfigError(f"config.json: 'layer_types' must list one entry per layer ({layers})")
        for t in layer_types:
            if t not in ("full_attention", "sliding_attention"):
                raise ConfigError(f"config.json: unknown layer type '{t}'")
        layer_types = tuple(layer_types)
    elif use_window and window is not None:
        first_windowed = _opt(raw, "max_window_layers", layers, int)
        layer_types = tuple("sliding_attention" if i >= first_windowed else "full_attention" for i in range(layers))
    else:
        layer_types = tuple("full_attention" for _ in range(layers))
    if "sliding_attention" in layer_types:
        if window is None or window <= 0:
            raise ConfigError("config.json: a layer is 'sliding_attention' but 'sliding_window' is not a positive integer")
    else:
        window = None
    eos = raw.get("eos_token_id")
    if eos is None:
        eos_ids: Tuple[int, ...] = ()
    elif isinstance(eos, int) and not isinstance(eos, bool):
        eos_ids = (eos,)
    elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
        eos_ids = tuple(eos)
    else:
        raise ConfigError(f"config.json: 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
    return Qwen3Config(
        vocab_size=_need(raw, "vocab_size"),
        hidden_size=hidden,
        intermediate_size=_need(raw, "intermediate_size"),
        num_hidden_layers=layers,
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        head_dim=head_dim,
        rms_norm_eps=_opt(raw, "rms_norm_eps", 1e-6, float),        # src/iian/arch/qwen3.cpp:17
        rope_theta=_opt(raw, "rope_theta", 10000.0, float),          # src/iian/model_loader.cpp:80
        max_position_embeddings=_need(raw, "max_position_embeddings"),
        tie_word_embeddings=_opt(raw, "tie_word_embeddings", False, bool),
        sliding_window=window,
        layer_types=layer_types,
        hidden_act=act,
        eos_token_ids=eos_ids,
    )


@register_architecture
class Qwen3(Architecture):
    name = "Qwen3ForCausalLM"

    def load_config(self, raw: Mapping[str, Any]) -> Qwen3Config:
        return qwen3_config_from_dict(raw)

    def config_to_dict(self, c: Qwen3Config) -> Dict[str, Any]:
        windowed = "sliding_attention" in c.layer_types
        d: Dict[str, Any] = {
            "architectures": [self.name],
            "model_type": "qwen3",
            "vocab_size": c.vocab_size,
            "hidden_size": c.hidden_size,
            "intermediate_size": c.intermediate_size,
            "num_hidden_layers": c.num_hidden_layers,
            "num_attention_heads": c.num_attention_heads,
            "num_key_value_heads": c.num_key_value_heads,
            "head_dim": c.head_dim,
            "hidden_act": c.hidden_act,
            "rms_norm_eps": c.rms_norm_eps,
            "rope_theta": c.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": c.max_position_embeddings,
            "tie_word_embeddings": c.tie_word_embeddings,
            "attention_bias": False,
            "use_sliding_window": windowed,
            "sliding_window": c.sliding_window if windowed else None,
        }
        if windowed:
            d["layer_types"] = list(c.layer_types)
        if c.eos_token_ids:
            d["eos_token_id"] = c.eos_token_ids[0] if len(c.eos_token_ids) == 1 else list(c.eos_token_ids)
        return d

    def build_spec(self, c: Qwen3Config) -> ModelSpec:
        def norm(size: int) -> PartSpec:
            return PartSpec("rms_norm", {"size": size, "eps": c.rms_norm_eps})

        layers = []
        for i in range(c.num_hidden_layers):
            rotary = PartSpec("rotary", {
                "dim": c.head_dim,                 # whole head rotates (qwen3.cpp:66)
                "base": c.rope_theta,
                "style": "neox",                   # qwen3.cpp:106
                "max_position": c.max_position_embeddings,
            })
            mixer = PartSpec("attention", {
                "hidden_size": c.hidden_size,
                "num_heads": c.num_attention_heads,
                "num_kv_heads": c.num_key_value_heads,
                "head_dim": c.head_dim,
                "scale": 1.0 / math.sqrt(c.head_dim),   # qwen3.cpp:72
                "qk_norm": True,
                "qk_norm_eps": c.rms_norm_eps,          # one eps for all norm sites
                "window": c.window_of_layer(i),
                "position": rotary,
            })
            ffn = PartSpec("gated_mlp", {
                "hidden_size": c.hidden_size,
                "intermediate_size": c.intermediate_size,
                "activation": c.hidden_act,
            })
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn,
                                    mixer_norm=norm(c.hidden_size), feed_forward_norm=norm(c.hidden_size)))
        return ModelSpec(
            hidden_size=c.hidden_size,
            vocab_size=c.vocab_size,
            max_position=c.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}),
            layers=tuple(layers),
            order=tuple(LayerCall(layer=i, cache=i) for i in range(c.num_hidden_layers)),
            final_norm=norm(c.hidden_size),
            head=PartSpec("lm_head", {"hidden_size": c.hidden_size, "vocab_size": c.vocab_size,
                                      "tied": c.tie_word_embeddings}),
        )

    _LAYER_SCOPES = {
        "mixer": "self_attn",
        "feed_forward": "mlp",
        "mixer_norm": "input_layernorm",
        "feed_forward_norm": "post_attention_layernorm",
    }

    def tensor_name(self, scope: tuple, local: str) -> str:
        if scope[0] == "embedding":
            return f"model.embed_tokens.{local}"
        if scope[0] == "final_norm":
            return f"model.norm.{local}"
        if scope[0] == "head":
            return f"lm_head.{local}"
        if scope[0] == "layer":
            return f"model.layers.{scope[1]}.{self._LAYER_SCOPES[scope[2]]}.{local}"
        raise KeyError(scope)
