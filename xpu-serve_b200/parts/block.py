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
the kernel side is csrc/gemm_small_m.cu). Parts opt in with `fuses_norm`.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import registry
from ..ops import lib as ops


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

    def __init__(self, stream: "ResidualStream", next_w: Optional[torch.Tensor]):
        self.stream, self.next_w = stream, next_w

    def product(self, act: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        st = self.stream
        rt = st.rt
        st.flush()
        if not rt.few_rows(act, w):
            st._pre = None
            st.add(rt.linear(act, w, "branch_out", bias), None, 0.0)
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
        self._pending = None      # (branch, post_w, eps_post)
        self._pre = None          # (norm weight, stream * weight, sums of squares) left by the last fused product
        self._flip = 0

    def add(self, branch: torch.Tensor, post_w: Optional[torch.Tensor], eps_post: float) -> None:
        if self._pending is not None:
            self.flush()
        self._pending = (branch, post_w, eps_post)

    def flush(self) -> None:
        if self._pending is not None:
            m, post_w, eps_post = self._pending
            ops.add_rmsnorm(self.h, m, post_w, None, None, None, eps_post, eps_post)
            self._pending = None
            self._pre = None

    def fuses(self) -> bool:
        """Whether this step's products between norms can carry the norm (few rows, bfloat16)."""
        rt = self.rt
        return (rt.mode == "bfloat16" and rt.fuse_norms and self.h.shape[0] <= rt.small_m and self.h.shape[1] % 8 == 0)

    def sink(self, next_w: Optional[torch.Tensor]) -> StreamSink:
        return StreamSink(self, next_w)

    def norm_input(self, w: torch.Tensor, eps: float, lazy: bool):
        """What a part reads: the normed stream, or (lazy, and the last fused product prepared for this very
        weight) the stream times the weight with its row scale pending."""
        if lazy and self._pending is None and self._pre is not None and self._pre[0] is w:
            return Prenormed(self._pre[1], self._pre[2], self.h.shape[1], eps)
        return self.norm(w, eps)

    def norm(self, w: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """RMSNorm of the stream (after any pending branch joined it), in the activation type.
        With `rows`, only those rows, packed."""
        n = self.h.shape[0] if rows is None else rows.numel()
        self._flip ^= 1
        y = self.rt.ws.get(f"normed{self._flip}", (n, self.h.shape[1]), self.rt.act_dtype)
        m, post_w, eps_post = self._pending if self._pending is not None else (None, None, eps)
        ops.add_rmsnorm(self.h, m, post_w, w, y, rows, eps, eps_post)
        if self._pending is not None:
            self._pre = None
        self._pending = None
        return y


class Block:
    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        """`weights`: this layer's tensors by their names under the layer's prefix."""
        self.spec, self.rt = spec, rt
        self.mixer = registry.mixer_class(spec.mixer.kind)(spec.mixer, weights, rt)
        self.ffn = registry.ffn_class(spec.ffn.kind)(spec.ffn, weights, rt)
        n = spec.names
        self.w_pre_mixer = rt.vector(weights[n["pre_mixer"]])
        self.w_pre_ffn = rt.vector(weights[n["pre_ffn"]])
        self.w_post_mixer = rt.vector(weights[n["post_mixer"]]) if spec.sandwich else None
        self.w_post_ffn = rt.vector(weights[n["post_ffn"]]) if spec.sandwich else None
        self.eps = spec.norm.eps

    def forward(self, stream: ResidualStream, step, cache, next_w: Optional[torch.Tensor] = None) -> None:
        """`next_w`: the weight of the norm that reads the stream after this block (the next block's, or the
        final norm's), for the fused path; None is always right."""
        fuse = stream.fuses() and not self.spec.sandwich
        if fuse and self.mixer.fuses_norm:
            x = stream.norm_input(self.w_pre_mixer, self.eps, lazy=True)
            self.mixer.forward(x, step, cache, into=stream.sink(self.w_pre_ffn))
        else:
            x = stream.norm(self.w_pre_mixer, self.eps)
            stream.add(self.mixer.forward(x, step, cache), self.w_post_mixer, self.eps)
        if fuse and self.ffn.fuses_norm:
            y = stream.norm_input(self.w_pre_ffn, self.eps, lazy=True)
            self.ffn.forward(y, step, into=stream.sink(next_w))
        else:
            y = stream.norm(self.w_pre_ffn, self.eps)
            stream.add(self.ffn.forward(y, step), self.w_post_ffn, self.eps)
