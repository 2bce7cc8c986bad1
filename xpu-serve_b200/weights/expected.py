"""The tensors a model spec expects, by full name, from its parts' declarations."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

from ..config.spec import ModelSpec
from ..parts.base import TensorSpec
from .. import registry


def layer_tensors(layer) -> Dict[str, TensorSpec]:
    """Relative names (under the layer's prefix) of one layer's tensors."""
    out: Dict[str, TensorSpec] = {}
    width = layer.norm.width
    keys = ["pre_mixer", "pre_ffn"] + (["post_mixer", "post_ffn"] if layer.sandwich else [])
    for key in keys:
        out[layer.names[key]] = TensorSpec((width,), init="ones", role="vector")
    out.update(registry.mixer_class(layer.mixer.kind).tensors(layer.mixer))
    out.update(registry.ffn_class(layer.ffn.kind).tensors(layer.ffn))
    return out


def expected_tensors(spec: ModelSpec, prefix: Optional[str] = None) -> Dict[str, TensorSpec]:
    """Full tensor names of the whole model, in a fixed order: embedding, final norm,
    head, then layer by layer. This order is also the order in which the random-weights
    mode draws tensors."""
    p = spec.prefixes[-1] if prefix is None else prefix
    out: Dict[str, TensorSpec] = {}
    out[p + spec.names["embed"]] = TensorSpec((spec.vocab, spec.hidden))
    out[p + spec.names["final_norm"]] = TensorSpec((spec.final_norm.width,), init="ones", role="vector")
    if not spec.tied_head:
        out[spec.names["head"]] = TensorSpec((spec.vocab, spec.hidden))
    for layer in spec.layers:
        for rel, ts in layer_tensors(layer).items():
            out[p + layer.prefix + rel] = ts
    return out


def probe_prefix(spec: ModelSpec, names: Sequence[str]) -> str:
    """The first of the spec's prefixes under which the embedding table is found
    (src/models/lfm3/lfm3_decoder.cpp:14-19)."""
    have = set(names)
    for p in spec.prefixes:
        if p + spec.names["embed"] in have:
            return p
    return spec.prefixes[-1]
