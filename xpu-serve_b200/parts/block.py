"""The arrangement of one decoder layer, and the residual stream it acts on.

    x = norm(h, pre_mixer);  h = h + post_mixer(mixer(x))
    y = norm(h, pre_ffn);    h = h + post_ffn(ffn(y))

where the post norms are RMSNorms when the layer is a sandwich and the identity
otherwise (src/models/lfm3/lfm3_decoder.cpp:78-90). The stream is float32. Adding a
branch is deferred until the next norm reads the stream, so that one kernel adds the
branch (normed or not), writes the sum back and produces the next normed input.

Decode steps (few rows, bfloat16, no sandwich norms) go without that kernel: the product that
ends a branch adds its result to the stream in its epilogue and leaves, beside it, the stream
times the next norm's weight and per-tile sums of squares; the product that starts the next
branch reads those and scales its result by each row's 1 / rms (`Prenormed`, `StreamSink`;
the kernel side is csrc/gemm_small_m.cu). Parts opt in with `fuses_norm`; it applies to norms that
say `carried` (RMSNorm).

The norms are parts too (parts/norm.py, registry.register_norm): the stream only calls their
`add_norm`. The arrangement itself is registered (`registry.register_arrangement`): `Block` is
"pre_norm"; another wiring of the same parts (post-norm, mixer and feed-forward side by side) is
another class with the same five members: tensors(layer), cache_need(layer), __init__(layer,
weights, rt), forward(stream, step, cache, next_norm), first_norm.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import registry
from .base import Norm, TensorSpec


class Prenormed:
    """The stream times a norm's weight, in bfloat16, with the sums of squares from which the product
    that reads it forms each row's 1 / sqrt(mean square + eps). Only `rt.linear` and
    `rt.few_rows_product` know what to do with it."""

    def __init__(self, x: torch.Tensor, ssq: torch.Tensor, width: int, eps: float):
        self.x, self.ssq, self.width, self.eps = x, ssq, width, eps

    @property
    def shape(self):
        return self.x.shape


class StreamSink:
    """Where a part's last product goes when it fuses: into the stream, inside the product's kernel."""

    def __init__(self, stream: "ResidualStream", next_norm: Optional[Norm]):
        """`next_norm`: the norm that reads the stream next, if the products can carry it (an RMSNorm)."""
        self.stream = stream
        self.next_w = next_norm.w if next_norm is not None and next_norm.carried else None

    def product(self, act: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        st = self.stream
        rt = st.rt
        st.flush()
        if not rt.few_rows(act, w):
            st._pre = None
            st.add(rt.linear(act, w, "branch_out", bias))
            return
        M, N = st.h.shape
        if self.next_w is None:
            rt.few_rows_product(act, w, None, bias, residual=st.h)
            st._pre = None
            return
        st._flip ^= 1
        nx = rt.ws.get(f"prenormed{st._flip}", (M, N), torch.bfloat16)
        ssq = rt.ws.get(f"ssq{st._flip}", ((N + 15) // 16, 16), torch.float32)
        rt.few_rows_product(act, w, None, bias, residual=st.h, next_w=self.next_w, next_x=nx, out_ssq=ssq)
        st._pre = (self.next_w, nx, ssq)


class ResidualStream:
    def __init__(self, h: torch.Tensor, rt):
        self.h, self.rt = h, rt
        self._pending = None      # (branch, the norm it passes through before it joins the stream, or None)
        self._pre = None          # (norm weight, stream * weight, sums of squares) left by the last fused product
        self._flip = 0
        self._plain_add: Optional[Norm] = None

    def add(self, branch: torch.Tensor, post: Optional[Norm] = None) -> None:
        if self._pending is not None:
            self.flush()
        self._pending = (branch, post)

    def flush(self, norm: Optional[Norm] = None) -> None:
        """Joins the pending branch to the stream now. `norm`: any norm of the model (its `add_norm` does the
        sum); without one the last norm that read the stream is used."""
        if self._pending is not None:
            m, post = self._pending
            norm = norm or post or self._plain_add
            if norm is None:
                raise RuntimeError("a branch is pending but no norm has read the stream yet")
            norm.add_norm(self.h, m, post, None, None)
            self._pending = None
            self._pre = None

    def fuses(self) -> bool:
        """Whether products of this step can add their result to the stream themselves and carry a norm across (few
        rows, bfloat16); which of them do is then asked part by part (`takes_prenormed`, `StreamSink.product`)."""
        rt = self.rt
        return (rt.mode == "bfloat16" and rt.fuse_norms and self.h.shape[0] <= max(rt.small_m, rt.narrow_m)
                and self.h.shape[1] % 8 == 0)

    def sink(self, next_norm: Optional[Norm]) -> StreamSink:
        return StreamSink(self, next_norm)

    def norm_input(self, norm: Norm, lazy: bool):
        """What a part reads: the normed stream, or (lazy, and the last fused product prepared for this very
        norm) the stream times the norm's weight with its row scale pending."""
        if (lazy and norm.carried and self._pending is None and self._pre is not None and self._pre[0] is norm.w):
            return Prenormed(self._pre[1], self._pre[2], self.h.shape[1], norm.eps)
        return self.norm(norm)

    def norm(self, norm: Norm, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`norm` of the stream (after any pending branch joined it), in the activation type.
        With `rows`, only those rows, packed."""
        n = self.h.shape[0] if rows is None else rows.numel()
        self._flip ^= 1
        y = self.rt.ws.get(f"normed{self._flip}", (n, self.h.shape[1]), self.rt.act_dtype)
        m, post = self._pending if self._pending is not None else (None, None)
        norm.add_norm(self.h, m, post, y, rows)
        if self._pending is not None:
            self._pre = None
        self._pending = None
        self._plain_add = norm
        return y


class Block:
    """The pre-norm arrangement (with optional sandwich norms)."""
    kind = "pre_norm"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, layer) -> Dict[str, TensorSpec]:
        """Relative names (under the layer's prefix) of the layer's tensors: its norms', its mixer's, its
        feed-forward's."""
        out: Dict[str, TensorSpec] = {}
        norm_cls = registry.norm_class(layer.norm.kind)
        keys = ["pre_mixer", "pre_ffn"] + (["post_mixer", "post_ffn"] if layer.sandwich else [])
        for key in keys:
            out.update(norm_cls.tensors(layer.norm, layer.names[key]))
        out.update(registry.mixer_class(layer.mixer.kind).tensors(layer.mixer))
        out.update(registry.ffn_class(layer.ffn.kind).tensors(layer.ffn))
        return out

    @classmethod
    def cache_need(cls, layer):
        return registry.mixer_class(layer.mixer.kind).cache_need(layer.mixer)

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        """`weights`: this layer's tensors by their names under the layer's prefix."""
        self.spec, self.rt = spec, rt
        self.mixer = registry.mixer_class(spec.mixer.kind)(spec.mixer, weights, rt)
        self.ffn = registry.ffn_class(spec.ffn.kind)(spec.ffn, weights, rt)
        n = spec.names
        norm_cls = registry.norm_class(spec.norm.kind)
        self.pre_mixer = norm_cls(spec.norm, weights, n["pre_mixer"], rt)
        self.pre_ffn = norm_cls(spec.norm, weights, n["pre_ffn"], rt)
        self.post_mixer = norm_cls(spec.norm, weights, n["post_mixer"], rt) if spec.sandwich else None
        self.post_ffn = norm_cls(spec.norm, weights, n["post_ffn"], rt) if spec.sandwich else None
        self.first_norm = self.pre_mixer      # the norm that reads the stream first: what the block before may prepare

    def forward(self, stream: ResidualStream, step, cache, next_norm: Optional[Norm] = None) -> None:
        """`next_norm`: the norm that reads the stream after this block (the next block's first, or the
        final norm), for the fused path; None is always right."""
        fuse = stream.fuses() and not self.spec.sandwich and self.pre_mixer.carried
        rows = stream.h.shape[0]
        # (a part whose first product runs elsewhere at this number of rows gets the normed tensor, and the product
        # before it does not prepare the norm's input for it; its last product may still add to the stream itself)
        ffn_lazy = fuse and self.ffn.fuses_norm and self.ffn.takes_prenormed(rows)
        if fuse and self.mixer.fuses_norm:
            x = stream.norm_input(self.pre_mixer, lazy=self.mixer.takes_prenormed(rows))
            self.mixer.forward(x, step, cache, into=stream.sink(self.pre_ffn if ffn_lazy else None))
        else:
            x = stream.norm(self.pre_mixer)
            stream.add(self.mixer.forward(x, step, cache), self.post_mixer)
        if fuse and self.ffn.fuses_norm:
            y = stream.norm_input(self.pre_ffn, lazy=ffn_lazy)
            self.ffn.forward(y, step, into=stream.sink(next_norm))
        else:
            y = stream.norm(self.pre_ffn)
            stream.add(self.ffn.forward(y, step), self.post_ffn)


registry.register_arrangement(Block.kind, Block)
