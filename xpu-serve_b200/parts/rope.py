"""Rotary position encoding as a table of (cos, sin) per position and channel pair.

Pair i couples channels i and i + head_dim/2 (rotate-half); inv_freq[i] is the float32
value of theta^(-2i/head_dim) for the first `pairs` pairs and 0 beyond them, so the
unrotated tail of a partially rotated head passes through unchanged
(src/models/common/blocks.cpp:131-141). The angle pos * inv_freq and its cos and sin are
formed in float64, as the reference's CPU backend forms them
(src/backend/cpu_ref/ops.cpp:383-387), and stored as float32: a float32 angle alone would
be off by up to pos * 2^-24 rad.

A position encoding of another kind registers a class with the same two methods; the
attention kernels only see the table.
"""
from __future__ import annotations

import torch

from .. import registry


class RotaryTable:
    kind = "rope"

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.key = ("rope", spec.head_dim, float(spec.theta), spec.pairs)

    def inv_freq(self) -> torch.Tensor:
        s = self.spec
        i = torch.arange(s.head_dim // 2, dtype=torch.float64)
        inv = (1.0 / torch.pow(torch.tensor(float(s.theta), dtype=torch.float64), 2.0 * i / s.head_dim))
        inv = inv.to(torch.float32)
        inv[s.pairs:] = 0.0
        return inv

    def table(self, n_positions: int) -> torch.Tensor:
        """[n_positions or more, head_dim / 2, 2] float32 on the device."""
        have = self.rt.shared.get(self.key)
        if have is not None and have.shape[0] >= n_positions:
            return have
        inv = self.inv_freq().to(device=self.rt.device, dtype=torch.float64)
        pos = torch.arange(n_positions, dtype=torch.float64, device=self.rt.device)
        angle = pos[:, None] * inv[None, :]
        table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()
        if have is not None:     # a captured graph may still read the shorter table: keep it alive
            self.rt.shared.setdefault(("kept",), []).append(have)
        self.rt.shared[self.key] = table
        return table


registry.register_position(RotaryTable.kind, RotaryTable)
