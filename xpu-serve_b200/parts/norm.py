"""RMSNorm over the last dimension, x * (mean(x^2) + eps)^(-1/2) * w, no +1 offset, in float32
(src/graph/graph.h:57, src/backend/cpu_ref/ops.cpp:260-281). One kernel adds a pending branch to
the stream (through the branch's own RMSNorm when the layer is a sandwich), writes the sum back
and produces the normed rows; in decode steps the few-row products carry this norm across
themselves instead (parts/block.py)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import registry
from ..ops import lib as ops
from .base import Norm


class RMSNorm(Norm):
    kind = "rmsnorm"
    carried = True

    def __init__(self, spec, weights, weight_name: str, rt):
        super().__init__(spec, weights, weight_name, rt)
        self.w = rt.vector(weights[weight_name])
        self.eps = float(spec.eps)

    def normed(self, x: torch.Tensor) -> torch.Tensor:
        h = x.float().contiguous()
        y = torch.empty(h.shape, dtype=self.rt.act_dtype, device=h.device)
        ops.add_rmsnorm(h, None, None, self.w, y, None, self.eps, self.eps)
        return y

    def add_norm(self, h, branch, post: Optional[Norm], y, rows) -> None:
        if post is not None and not isinstance(post, RMSNorm):
            return super().add_norm(h, branch, post, y, rows)
        ops.add_rmsnorm(h, branch, None if post is None else post.w, self.w if y is not None else None, y, rows,
                        self.eps, self.eps if post is None else post.eps)


registry.register_norm(RMSNorm.kind, RMSNorm)
