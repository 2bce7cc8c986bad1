"""SwiGLU feed-forward: down(silu(gate y) * up y) (src/models/common/blocks.cpp:23-27). The
gate and up weights are stacked at load so that one matrix product gives both."""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import FeedForward, TensorSpec


class SwiGLU(FeedForward):
    kind = "swiglu"

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        return {n["gate"]: TensorSpec((spec.intermediate, spec.hidden)),
                n["up"]: TensorSpec((spec.intermediate, spec.hidden)),
                n["down"]: TensorSpec((spec.hidden, spec.intermediate))}

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_gate_up = rt.matrix(torch.cat([weights[n["gate"]].to(torch.float32),
                                              weights[n["up"]].to(torch.float32)], 0))
        self.w_down = rt.matrix(weights[n["down"]])

    def forward(self, y: torch.Tensor, step) -> torch.Tensor:
        rt, F = self.rt, self.spec.intermediate
        gu = rt.linear(y, self.w_gate_up, "ffn_gate_up")
        act = rt.ws.get("ffn_act", (y.shape[0], F), rt.act_dtype)
        ops.silu_mul(gu, act)
        return rt.linear(act, self.w_down, "ffn_out")


registry.register_ffn(SwiGLU.kind, SwiGLU)
