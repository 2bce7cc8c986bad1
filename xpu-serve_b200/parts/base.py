"""What every part declares: its tensors, and (for mixers) what it keeps per sequence.

A part is a class built from a spec (config/spec.py) whose `kind` names it in the
registry. Declaring tensors is separate from running: `tensors(spec)` needs no GPU, so
a model folder can be checked, or written with random weights, on any machine.

Interfaces
----------
Mixer:        tensors(spec) -> {relative name: TensorSpec}
              cache_need(spec) -> KVNeed | StateNeed | None
              __init__(spec, weights, rt)          weights: {relative name: device tensor}
              forward(x, step, cache) -> [tokens, hidden]   x is the normed stream
FeedForward:  tensors(spec); __init__(spec, weights, rt); forward(y, step) -> [tokens, hidden]
Position:     __init__(spec, rt, max_position); table() -> device tensors the mixer passes
              to its kernels
Optional, for decode steps (few rows): a part whose class sets `fuses_norm = True` takes
`forward(x, step, cache, into=None)` (feed-forward: `forward(y, step, into=None)`). Its x may then be
a parts.block.Prenormed (the stream times the norm's weight, with the row scale still to apply),
which it may hand to `rt.linear` / `rt.few_rows_product` only; and when `into` is given it sends its
last product through `into.product(act, w, bias)` (which adds it to the stream inside the product's
kernel) and returns None. Parts without the flag get the normed tensor and return their branch.
`step` is engine.step.StepContext (which tokens belong to which sequence, where each
sequence stands), `cache` the view of this call's storage (cache/views.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    init: str = "normal"     # random-weights mode: "normal" N(0, std) | "ones" | "zeros"
    role: str = "matrix"     # "matrix": held in the compute dtype; "vector": held in float32


@dataclass(frozen=True)
class KVNeed:
    """Keys and values for every cached position (window 0) or the last `window` of them."""
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per sequence, zero at a sequence's start."""
    shape: Tuple[int, ...]
    dtype: str = "compute"   # "compute": the activation dtype; "float32"


class Part:
    kind: str = ""
    fuses_norm: bool = False    # see the module text: takes a Prenormed input and an `into` sink

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        return {}


class Mixer(Part):
    @classmethod
    def cache_need(cls, spec):
        return None

    def forward(self, x, step, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, y, step):
        raise NotImplementedError
