"""The arrangement of one decoder layer, and the residual stream it acts on.

    x = norm(h, pre_mixer);  h = h + post_mixer(mixer(x))
    y = norm(h, pre_ffn);    h = h + post_ffn(ffn(y))

where the post norms are RMSNorms when the layer is a sandwich and the identity
otherwise (src/models/lfm3/lfm3_decoder.cpp:78-90). The stream is float32. Adding a
branch is deferred until the next norm reads the stream, so that one kernel adds the
branch (normed or not), writes the sum back and produces the next normed input.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import registry
from ..ops import lib as ops


class ResidualStream:
    def __init__(self, h: torch.Tensor, rt):
        self.h, self.rt = h, rt
        self._pending = None      # (branch, post_w, eps_post)
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

    def norm(self, w: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """RMSNorm of the stream (after any pending branch joined it), in the activation type.
        With `rows`, only those rows, packed."""
        n = self.h.shape[0] if rows is None else rows.numel()
        self._flip ^= 1
        y = self.rt.ws.get(f"normed{self._flip}", (n, self.h.shape[1]), self.rt.act_dtype)
        m, post_w, eps_post = self._pending if self._pending is not None else (None, None, eps)
        ops.add_rmsnorm(self.h, m, post_w, w, y, rows, eps, eps_post)
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

    def forward(self, stream: ResidualStream, step, cache) -> None:
        x = stream.norm(self.w_pre_mixer, self.eps)
        stream.add(self.mixer.forward(x, step, cache), self.w_post_mixer, self.eps)
        y = stream.norm(self.w_pre_ffn, self.eps)
        stream.add(self.ffn.forward(y, step), self.w_post_ffn, self.eps)
