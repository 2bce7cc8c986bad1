"""Typed configuration of LFM3, read from config.json's own keys.

Keys and defaults follow src/models/lfm3/lfm3_config.cpp:42-99. Three switches that
the reference refuses are options here (`use_sandwich_norm` false, an untied head,
`conv_bias`), one is added (`attn_head_gate`; the reference always has the gate,
src/models/common/blocks.cpp:182), and `layer_types` also accepts "attn" for
"full_attention". A flat `rope_theta` stands for a `rope_parameters` entry that rotates
the whole head.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .json_util import (ConfigError, get_bool_or, get_float, get_float_or, get_int,
                        get_int_list, get_int_or, get_str, get_str_or)
from .spec import (AttentionSpec, LayerCall, LayerSpec, ModelSpec, NormSpec, RopeSpec,
                   ShortConvSpec, SwiGLUSpec)

CONV = "conv"
FULL = "full_attention"
SLIDING = "sliding_attention"
_LAYER_ALIASES = {"conv": CONV, "full_attention": FULL, "attn": FULL, "attention": FULL,
                  "sliding_attention": SLIDING}


@dataclass(frozen=True)
class Lfm3Rope:
    theta: float
    partial_rotary_factor: float = 1.0

    def pairs(self, head_dim: int) -> int:
        # int(factor * head_dim) / 2, src/models/lfm3/lfm3_config.cpp:20
        return int(self.partial_rotary_factor * float(head_dim)) // 2


@dataclass(frozen=True)
class Lfm3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    norm_eps: float
    max_position_embeddings: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    conv_L_cache: int
    layer_types: Tuple[str, ...]
    rope: Dict[str, Lfm3Rope] = field(default_factory=dict)   # by FULL / SLIDING
    sliding_window: int = 0
    conv_bias: bool = False
    use_sandwich_norm: bool = True
    attn_head_gate: bool = True
    tie_word_embeddings: bool = True
    initializer_range: float = 0.02
    eos_token_id: Tuple[int, ...] = ()
    model_type: str = "lfm3"

    # ---------------------------------------------------------------- parsing
    @staticmethod
    def text_config(cfg: dict) -> dict:
        """All of an lfm3 config.json, the text_config of an lfm3_vl one
        (src/models/lfm3/lfm3_config.cpp:28-40)."""
        mt = get_str(cfg, "model_type", "config.json")
        if mt == "lfm3":
            return cfg
        if mt != "lfm3_vl":
            raise ConfigError(f"lfm3: model_type '{mt}' is not supported (lfm3, lfm3_vl are)")
        text = cfg.get("text_config")
        if not isinstance(text, dict):
            raise ConfigError("config.json: an lfm3_vl checkpoint without a text_config")
        tt = get_str_or(text, "model_type", "lfm3", "config.json text_config")
        if tt != "lfm3":
            raise ConfigError(f"config.json: text_config model_type '{tt}' is not supported (lfm3 is)")
        return text

    @classmethod
    def from_json(cls, cfg: dict) -> "Lfm3Config":
        t = cls.text_config(cfg)
        w = "config.json"
        tied = get_bool_or(t, "tie_embedding", get_bool_or(t, "tie_word_embeddings", True, w), w)
        hidden = get_int(t, "hidden_size", w)
        heads = get_int(t, "num_attention_heads", w)
        kv_heads = get_int(t, "num_key_value_heads", w)
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads != 0:
            raise ConfigError(f"{w}: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        head_dim = get_int_or(t, "head_dim", hidden // heads, w)
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"{w}: head_dim {head_dim} must be even")
        kernel = get_int_or(t, "conv_L_cache", 7, w)
        if kernel < 2:
            raise ConfigError(f"{w}: conv_L_cache must be at least 2")
        n_layers = get_int(t, "num_hidden_layers", w)

        lt = t.get("layer_types")
        if not isinstance(lt, list):
            raise ConfigError(f"{w}: missing layer_types")
        kinds: List[str] = []
        for s in lt:
            if not isinstance(s, str):
                raise ConfigError(f"{w}: layer_types must be a list of strings")
            if s not in _LAYER_ALIASES:
                raise ConfigError(f"{w}: unknown layer type '{s}'")
            kinds.append(_LAYER_ALIASES[s])
        if len(kinds) != n_layers:
            raise ConfigError(f"{w}: layer_types has {len(kinds)} entries for {n_layers} layers")

        rope: Dict[str, Lfm3Rope] = {}
        needed = [k for k in (FULL, SLIDING) if k in kinds]
        if needed:
            rp = t.get("rope_parameters")
            for kind in needed:
                if isinstance(rp, dict) and isinstance(rp.get(kind), dict):
                    r = rp[kind]
                    rw = f"{w} rope_parameters.{kind}"
                    rtype = get_str_or(r, "rope_type", "default", rw)
                    if rtype != "default":
                        raise ConfigError(f"{rw}: rope_type '{rtype}' is not supported (supported: default)")
                    entry = Lfm3Rope(get_float(r, "rope_theta", rw),
                                     get_float_or(r, "partial_rotary_factor", 1.0, rw))
                elif isinstance(rp, dict) and "rope_theta" in rp and not any(
                        isinstance(v, dict) for v in rp.values()):
                    # one flat rope_parameters object for every attention layer
                    rw = f"{w} rope_parameters"
                    entry = Lfm3Rope(get_float(rp, "rope_theta", rw),
                                     get_float_or(rp, "partial_rotary_factor", 1.0, rw))
                elif rp is None and "rope_theta" in t:
                    entry = Lfm3Rope(get_float(t, "rope_theta", w), 1.0)
                elif rp is None:
                    raise ConfigError(f"{w}: missing rope_parameters")
                else:
                    raise ConfigError(f"{w}: rope_parameters has no entry for the {kind} layers")
                pairs = entry.pairs(head_dim)
                if not (entry.theta > 0 and 1 <= pairs <= head_dim // 2):
                    raise ConfigError(f"{w} rope_parameters.{kind}: theta {entry.theta} and {pairs} "
                                      f"rotated pairs do not fit head_dim {head_dim}")
                rope[kind] = entry
        window = 0
        if SLIDING in kinds:
            window = get_int(t, "sliding_window", w)
            if window <= 0:
                raise ConfigError(f"{w}: sliding_window must be positive")

        eos = tuple(get_int_list(cfg, "eos_token_id", w)) or tuple(get_int_list(t, "eos_token_id", w))
        c = cls(
            vocab_size=get_int(t, "vocab_size", w),
            hidden_size=hidden,
            intermediate_size=get_int(t, "intermediate_size", w),
            num_hidden_layers=n_layers,
            norm_eps=get_float(t, "norm_eps", w),
            max_position_embeddings=get_int(t, "max_position_embeddings", w),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            conv_L_cache=kernel,
            layer_types=tuple(kinds),
            rope=rope,
            sliding_window=window,
            conv_bias=get_bool_or(t, "conv_bias", False, w),
            use_sandwich_norm=get_bool_or(t, "use_sandwich_norm", True, w),
            attn_head_gate=get_bool_or(t, "attn_head_gate", True, w),
            tie_word_embeddings=tied,
            initializer_range=get_float_or(t, "initializer_range", 0.02, w),
            eos_token_id=eos,
        )
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "max_position_embeddings"):
            if getattr(c, name) <= 0:
                raise ConfigError(f"{w}: {name} must be positive")
        if not c.norm_eps > 0:
            raise ConfigError(f"{w}: norm_eps must be positive")
        return c

    def to_json(self) -> dict:
        """A config.json that from_json reads back to this configuration."""
        d = {
            "model_type": self.model_type,
            "architectures": ["Lfm3ForCausalLM"],
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "norm_eps": self.norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": self.conv_bias,
            "use_sandwich_norm": self.use_sandwich_norm,
            "attn_head_gate": self.attn_head_gate,
            "tie_word_embeddings": self.tie_word_embeddings,
            "initializer_range": self.initializer_range,
            "layer_types": list(self.layer_types),
        }
        if self.rope:
            d["rope_parameters"] = {
                kind: {"rope_type": "default", "rope_theta": r.theta,
                       "partial_rotary_factor": r.partial_rotary_factor}
                for kind, r in self.rope.items()}
        if self.sliding_window:
            d["sliding_window"] = self.sliding_window
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------- to a model spec
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(self.hidden_size, self.norm_eps)
        ffn = SwiGLUSpec(self.hidden_size, self.intermediate_size)
        layers = []
        for i, kind in enumerate(self.layer_types):
            if kind == CONV:
                mixer: object = ShortConvSpec(self.hidden_size, self.conv_L_cache, self.conv_bias)
            else:
                r = self.rope[kind]
                mixer = AttentionSpec(
                    hidden=self.hidden_size, heads=self.num_attention_heads,
                    kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                    qk_norm=True, qk_norm_eps=self.norm_eps,
                    position=RopeSpec(self.head_dim, r.theta, r.pairs(self.head_dim)),
                    window=self.sliding_window if kind == SLIDING else 0,
                    head_gate=self.attn_head_gate,
                    # 1/sqrt(head_dim), src/models/lfm3/lfm3_decoder.cpp:122
                    scale=1.0 / math.sqrt(float(self.head_dim)))
            layers.append(LayerSpec(prefix=f"layers.{i}.", mixer=mixer, ffn=ffn, norm=norm,
                                    sandwich=self.use_sandwich_norm))
        spec = ModelSpec(
            arch="lfm3", vocab=self.vocab_size, hidden=self.hidden_size,
            max_position=self.max_position_embeddings, layers=tuple(layers),
            order=tuple(LayerCall(i) for i in range(len(layers))),
            final_norm=norm, tied_head=self.tie_word_embeddings,
            init_std=self.initializer_range,
            # lfm3_vl keeps the decoder under model.language_model. (lfm3_decoder.cpp:14-19)
            prefixes=("model.language_model.", "model."))
        spec.validate()
        return spec
