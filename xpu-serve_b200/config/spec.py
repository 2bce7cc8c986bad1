"""Architecture-neutral description of a decoder: what each layer is made of.

An architecture's typed configuration (config/lfm3.py for LFM3) is turned into a
`ModelSpec`: a list of `LayerSpec`s, each naming its mixer, its feed-forward and its
norms by `kind` with every size, constant and tensor name as a field, plus the order
in which the layers run. The engine builds parts from these specs through the part
registries (registry.py) and never looks at the architecture's own configuration, so
a part does not know which model it is in, and two layers of one model can use
different mixers and feed-forwards.

The reference expresses the same thing as a graph built once per model
(src/models/lfm3/lfm3_decoder.cpp:49-90); here the description is data and the step
function interprets it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary position encoding (src/models/common/blocks.cpp:131-141).

    Pair i couples channels i and i + head_dim/2; pairs i < `pairs` turn by
    pos * theta^(-2i/head_dim), the others by 0 (identity). `pairing` "interleaved": pair i couples
    channels 2i and 2i + 1 instead (LFM3 has "half"; the mixer that reads this brings such a checkpoint
    into the rotate-half order when it loads its weights, so the kernels know one order only).
    """
    head_dim: int
    theta: float
    pairs: int
    kind: str = "rope"
    pairing: str = "half"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a key/value cache (src/models/common/blocks.cpp:143-187)."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    qk_norm: bool            # RMSNorm over head_dim on q and k, before the position encoding
    qk_norm_eps: float
    position: Optional[RopeSpec]
    window: int              # 0: every earlier key is visible; W > 0: keys with pos - j < W
    head_gate: bool          # o[t, h, :] *= sigmoid((x Wg^T)[t, h])
    scale: float             # multiplies q.k before the softmax
    names: Dict[str, str] = field(default_factory=lambda: {
        "q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
        "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight",
        "gate": "self_attn.gate_proj.weight",
        "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight",
        "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias", "v_bias": "self_attn.v_proj.bias"})
    kind: str = "attention"
    qkv_bias: bool = False   # q, k and v projections with a bias each (LFM3 has none)


@dataclass(frozen=True)
class ShortConvSpec:
    """Gated causal depthwise convolution with a fixed-size state
    (src/models/lfm3/lfm3_decoder.cpp:94-111)."""
    hidden: int
    kernel: int              # taps; the state holds kernel - 1 rows per sequence
    bias: bool               # conv.conv.bias, in_proj.bias, out_proj.bias
    names: Dict[str, str] = field(default_factory=lambda: {
        "in": "conv.in_proj.weight", "conv": "conv.conv.weight", "out": "conv.out_proj.weight",
        "in_bias": "conv.in_proj.bias", "conv_bias": "conv.conv.bias", "out_bias": "conv.out_proj.bias"})
    kind: str = "short_conv"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate x) * up x) (src/models/common/blocks.cpp:23-27)."""
    hidden: int
    intermediate: int
    names: Dict[str, str] = field(default_factory=lambda: {
        "gate": "feed_forward.w1.weight", "up": "feed_forward.w3.weight",
        "down": "feed_forward.w2.weight"})
    kind: str = "swiglu"


@dataclass(frozen=True)
class NormSpec:
    """RMSNorm over the last dimension, x * (mean(x^2) + eps)^(-1/2) * w, no +1 offset
    (src/graph/graph.h:57, src/backend/cpu_ref/ops.cpp:260-281)."""
    width: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: h += post(mixer(pre(h))); h += post(ffn(pre(h)))
    (src/models/lfm3/lfm3_decoder.cpp:78-90). With `sandwich` false the post norms are
    the identity and their tensors are not read."""
    prefix: str              # tensor-name prefix under the model prefix, e.g. "layers.3."
    mixer: object            # a spec with a `kind`
    ffn: object              # a spec with a `kind`
    norm: NormSpec
    sandwich: bool
    names: Dict[str, str] = field(default_factory=lambda: {
        "pre_mixer": "operator_norm.weight", "post_mixer": "post_operator_norm.weight",
        "pre_ffn": "ffn_norm.weight", "post_ffn": "post_ffn_norm.weight"})
    kind: str = "pre_norm"   # the arrangement (registry.register_arrangement); the formula above is "pre_norm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the running order. `layer` indexes ModelSpec.layers (a layer may be
    called more than once; each call keeps its own cache). `cache_of` is the index, in
    the running order, of an earlier call whose cache this call's mixer reads instead
    of owning one."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    arch: str
    vocab: int
    hidden: int
    max_position: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tied_head: bool
    init_std: float = 0.02   # random-weights mode: matrices and tables ~ N(0, init_std)
    embed_scale: float = 1.0  # the embedding rows are multiplied by it (1: as stored, LFM3's)
    logit_cap: float = 0.0    # > 0: logits = cap * tanh(logits / cap) (0: none, LFM3's)
    prefixes: Tuple[str, ...] = ("model.",)   # tried in turn for "<prefix>embed_tokens.weight"
    names: Dict[str, str] = field(default_factory=lambda: {
        "embed": "embed_tokens.weight", "final_norm": "embedding_norm.weight",
        "head": "lm_head.weight"})   # "head" is looked up without the model prefix

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("the running order is empty")
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {call.layer} of {len(self.layers)}")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < i:
                    raise ValueError(f"order[{i}] reads the cache of call {call.cache_of}, which does not run before it")
                if self.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}] reads the cache of call {call.cache_of}, which owns none")
