"""The tensors a model spec expects, by full name, from its parts' declarations."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

from ..config.spec import ModelSpec
from ..parts.base import TensorSpec
from .. import registry


def layer_tensors(layer) -> Dict[str, TensorSpec]:
    """Relative names (under the layer's prefix) of one layer's tensors, as its arrangement declares them."""
    return registry.arrangement_class(layer.kind).tensors(layer)


def expected_tensors(spec: ModelSpec, prefix: Optional[str] = None) -> Dict[str, TensorSpec]:
    """Full tensor names of the whole model, in a fixed order: embedding, final norm,
    head, then layer by layer. This order is also the order in which the random-weights
    mode draws tensors."""
    p = spec.prefixes[-1] if prefix is None else prefix
    out: Dict[str, TensorSpec] = {}
    out[p + spec.names["embed"]] = TensorSpec((spec.vocab, spec.hidden))
    for rel, ts in registry.norm_class(spec.final_norm.kind).tensors(spec.final_norm, spec.names["final_norm"]).items():
        out[p + rel] = ts
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
