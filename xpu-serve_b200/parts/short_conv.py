"""Gated short convolution: out_proj(C * conv(B * x)) with [B | C | x] = in_proj(input), a
causal depthwise convolution over `kernel` positions whose last kernel - 1 inputs are the
sequence's fixed-size state (src/models/lfm3/lfm3_decoder.cpp:94-111).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import Mixer, StateNeed, TensorSpec


class ShortConvMixer(Mixer):
    kind = "short_conv"
    fuses_norm = True
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n, H = spec.names, spec.hidden
        out = {n["in"]: TensorSpec((3 * H, H)), n["conv"]: TensorSpec((H, 1, spec.kernel)),
               n["out"]: TensorSpec((H, H))}
        if spec.bias:
            out[n["in_bias"]] = TensorSpec((3 * H,), role="vector")
            out[n["conv_bias"]] = TensorSpec((H,), role="vector")
            out[n["out_bias"]] = TensorSpec((H,), role="vector")
        return out

    @classmethod
    def cache_need(cls, spec):
        return StateNeed((spec.kernel - 1, spec.hidden), "compute")

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.kernel < 2:
            raise ValueError("short_conv: the kernel needs at least 2 taps")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_in = rt.matrix(weights[n["in"]])
        self.w_out = rt.matrix(weights[n["out"]])
        # taps transposed to [kernel, hidden] so that neighbouring channels are neighbours in memory
        self.taps = rt.vector(weights[n["conv"]].reshape(spec.hidden, spec.kernel).t())
        self.b_in = rt.vector(weights[n["in_bias"]]) if spec.bias else None
        self.b_conv = rt.vector(weights[n["conv_bias"]]) if spec.bias else None
        self.b_out = rt.vector(weights[n["out_bias"]]) if spec.bias else None

    def takes_prenormed(self, rows: int) -> bool:
        return self.rt.few_rows_shape(rows, self.w_in) and self.w_in.shape[1] % 8 == 0

    def forward(self, x, step, cache, into=None) -> torch.Tensor:
        rt, H = self.rt, self.spec.hidden
        if cache is None or cache.storage is None or not cache.owner:
            raise RuntimeError("short_conv keeps its own state and cannot read another call's")
        y = rt.ws.get("conv_y", (x.shape[0], H), rt.act_dtype)
        if step.decode and rt.conv_behind_product(x, self.w_in, H):
            # one token a sequence: the convolution and the state's update run in the tail of the in_proj product
            bcx = rt.ws.get("conv_bcx", (x.shape[0], 3 * H), rt.act_dtype)
            rt.few_rows_product(x, self.w_in, bcx, self.b_in,
                                conv=dict(taps=self.taps, bias=self.b_conv, state=cache.storage, slots=step.slots, out=y))
            if into is not None:
                return into.product(y, self.w_out, self.b_out)
            return rt.linear(y, self.w_out, "mixer_out", self.b_out)
        bcx = rt.linear(x, self.w_in, "conv_bcx", self.b_in)
        ops.short_conv(bcx, self.taps, self.b_conv, cache.storage, step.seq_of_token, step.cu_seqlens, step.slots, y,
                       all_single=step.decode)
        if into is not None:
            return into.product(y, self.w_out, self.b_out)
        return rt.linear(y, self.w_out, "mixer_out", self.b_out)


registry.register_mixer(ShortConvMixer.kind, ShortConvMixer)
