"""SwiGLU feed-forward: down(silu(gate y) * up y) (src/models/common/blocks.cpp:23-27). The
gate and up weights are stacked at load so that one matrix product gives both. When the
width allows (a multiple of 8, bfloat16) they are stacked in blocks of 8 gate rows and the 8
up rows of the same outputs: the few-row product and, for long prompts, the tcgen05 product
then apply the activation in their epilogue and write silu(gate) * up directly."""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import FeedForward, TensorSpec


class SwiGLU(FeedForward):
    kind = "swiglu"
    fuses_norm = True
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        return {n["gate"]: TensorSpec((spec.intermediate, spec.hidden)),
                n["up"]: TensorSpec((spec.intermediate, spec.hidden)),
                n["down"]: TensorSpec((spec.hidden, spec.intermediate))}

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        self.spec, self.rt = spec, rt
        n = spec.names
        gate, up = weights[n["gate"]].to(torch.float32), weights[n["up"]].to(torch.float32)
        F, H = spec.intermediate, spec.hidden
        self.interleave = 8 if (rt.mode == "bfloat16" and F % 8 == 0) else 0
        if self.interleave:
            stacked = torch.stack([gate.view(F // 8, 8, H), up.view(F // 8, 8, H)], 1).reshape(2 * F, H)
        else:
            stacked = torch.cat([gate, up], 0)
        self.w_gate_up = rt.matrix(stacked)
        self.w_down = rt.matrix(weights[n["down"]])

    def takes_prenormed(self, rows: int) -> bool:
        return bool(self.interleave) and self.rt.few_rows_shape(rows, self.w_gate_up) and self.w_gate_up.shape[1] % 8 == 0

    def forward(self, y, step, into=None) -> torch.Tensor:
        rt, F = self.rt, self.spec.intermediate
        act = rt.ws.get("ffn_act", (y.shape[0], F), rt.act_dtype)
        if self.interleave and rt.few_rows(y, self.w_gate_up):
            rt.few_rows_product(y, self.w_gate_up, act, swiglu=True)
        elif self.interleave and rt.tensor_core_product(y, self.w_gate_up, fused=True):
            ops.gemm_tc(y, self.w_gate_up, act, epilogue=ops.EPI_SWIGLU)
        else:
            gu = rt.linear(y, self.w_gate_up, "ffn_gate_up")
            ops.silu_mul(gu, act, self.interleave)
        if into is not None:
            return into.product(act, self.w_down)
        return rt.linear(act, self.w_down, "ffn_out")


registry.register_ffn(SwiGLU.kind, SwiGLU)
