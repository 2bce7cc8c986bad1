"""What every part declares: its tensors, and (for mixers) what it keeps per sequence.

A part is a class built from a spec (config/spec.py) whose `kind` names it in the
registry. Declaring tensors is separate from running: `tensors(spec)` needs no GPU, so
a model folder can be checked, or written with random weights, on any machine.

Interfaces
----------
Mixer:        tensors(spec) -> {relative name: TensorSpec}
              cache_need(spec) -> None | KVNeed | StateNeed | a tuple of those (a mixer that keeps
                                  several things per sequence: a window of inputs and a running
                                  state, keys/values and a state, ...)
              __init__(spec, weights, rt)          weights: {relative name: device tensor}
              forward(x, step, cache) -> [tokens, hidden]   x is the normed stream; `cache` is the
                                  view of this call's storage (cache.CallView): `cache.storage`
                                  for one need, `cache[k].storage` for the k-th of several
FeedForward:  tensors(spec); __init__(spec, weights, rt); forward(y, step) -> [tokens, hidden]
Position:     __init__(spec, rt); table(n_positions) -> device tensor the mixer passes to its
              kernels
Norm:         tensors(spec, weight_name) -> {relative name: TensorSpec}
              __init__(spec, weights, weight_name, rt)
              normed(x) -> the normed rows of x, float32 or the activation type
              (optional) add_norm(h, branch, post, y, rows): h += post(branch); y = self(h[rows])
              in one pass; the base class does it in steps through `normed`
Arrangement   (of one layer: which norm feeds which part and how branches join the stream):
              tensors(layer) ; cache_need(layer) ; __init__(layer, weights, rt) ;
              forward(stream, step, cache, next_norm=None) ; `first_norm`
Optional, for decode steps (few rows): a part whose class sets `fuses_norm = True` takes
`forward(x, step, cache, into=None)` (feed-forward: `forward(y, step, into=None)`). Its x may then be
a parts.block.Prenormed (the stream times the norm's weight, with the row scale still to apply),
which it may hand to `rt.linear` / `rt.few_rows_product` only; and when `into` is given it sends its
last product through `into.product(act, w, bias)` (which adds it to the stream inside the product's
kernel) and returns None. Parts without the flag get the normed tensor and return their branch.
Such a part also says, per number of rows, whether the product that reads its input runs on the few-row kernel
(`takes_prenormed(rows)`): only then is it handed a Prenormed; otherwise it gets the normed tensor, and still `into`.
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
    # Whether the part's code for prompt steps can be captured in a CUDA graph that serves any lengths up to the step's
    # bounds (`step.fixed_shape`): no host-side loop over `step.q_lens_host`, no host sync, sizes from the tensors'
    # shapes and `step.max_q_len` only. The library's parts say yes; the model captures single-sequence prompt steps
    # only when every part of it does. (Decode steps must be capturable in any case.)
    fixed_shape_ok: bool = False

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        return {}

    def takes_prenormed(self, rows: int) -> bool:
        """Parts with `fuses_norm`: whether, for a step of `rows` rows, the product that reads the part's input runs on
        the few-row kernel, which alone can apply a norm's row scale (engine/runtime.py: Runtime.few_rows_shape)."""
        return False


class Mixer(Part):
    @classmethod
    def cache_need(cls, spec):
        return None

    def forward(self, x, step, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, y, step):
        raise NotImplementedError


class Norm(Part):
    """A normalisation over the last dimension. A new kind implements `tensors` and `normed`; `add_norm`
    (what the residual stream calls) then works through them. `carried` says whether the few-row products
    can carry this norm across themselves (RMSNorm only: see parts/block.py)."""
    carried: bool = False
    fixed_shape_ok = True       # `normed` works on tensors alone

    @classmethod
    def tensors(cls, spec, weight_name: str) -> Dict[str, TensorSpec]:
        return {weight_name: TensorSpec((spec.width,), init="ones", role="vector")}

    def __init__(self, spec, weights, weight_name: str, rt):
        self.spec, self.rt = spec, rt

    def normed(self, x):
        raise NotImplementedError

    def add_norm(self, h, branch, post: Optional["Norm"], y, rows) -> None:
        """h (the float32 stream) += post(branch) (branch alone without `post`); then y = self(h), of the
        rows `rows` only when given. `branch` or `y` may be None (no branch pending; only the sum wanted)."""
        if branch is not None:
            h.add_(post.normed(branch).float() if post is not None else branch.float())
        if y is not None:
            y.copy_(self.normed(h if rows is None else h.index_select(0, rows.long())))
