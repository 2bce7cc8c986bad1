"""One step's description on the device: which tokens run, whose they are, where they stand.

A step runs only the tokens it is given, packed one sequence after another. Sequences of
one step may have different lengths; each has its own slot, its own position offset
(the length its slot already holds) and its own page-table row. Everything the kernels
need is laid out in ONE int32 buffer on the host (pinned) and copied to the device with
one transfer:

    tokens[T] positions[T] seq_of_token[T] cu_seqlens[n+1] slots[n] kv_lens[n] want_rows[W]
    then one page table [n, P_g] per key/value group

The reference's step takes `token_ids[T]` and `positions[T]` for its single sequence
(src/models/lfm3/lfm3_decoder.cpp:26-47); the rest is what batching adds.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


def _round4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class StepContext:
    n_seqs: int
    n_tokens: int
    decode: bool                 # every sequence brings exactly one token
    max_q_len: int
    max_kv_len: int
    page_size: int
    max_positions: int           # the longest a sequence of this cache can get (rotary tables cover it)
    tokens: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    cu_seqlens: torch.Tensor
    slots: torch.Tensor
    kv_lens: torch.Tensor        # length of each sequence after this step
    want_rows: torch.Tensor
    page_tables: Dict[int, torch.Tensor] = field(default_factory=dict)
    q_lens_host: Optional[np.ndarray] = None
    starts_host: Optional[np.ndarray] = None


class StepStager:
    """Owns the pinned host buffer and the device buffer that a step's description goes through."""

    def __init__(self, device, capacity: int = 1 << 16):
        self.device = torch.device(device)
        self._host = None
        self._dev = None
        self._event = None
        self.last_h2d_bytes = 0
        self._grow(capacity)

    def _grow(self, n: int) -> None:
        pin = self.device.type == "cuda"
        self._host = torch.empty(n, dtype=torch.int32, pin_memory=pin)
        self._dev = torch.empty(n, dtype=torch.int32, device=self.device)
        self._np = self._host.numpy()

    def stage(self, cache, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
              want: Sequence[Sequence[int]], starts: np.ndarray) -> StepContext:
        n = len(slots)
        q_lens = np.fromiter((len(t) for t in token_lists), dtype=np.int64, count=n)
        T = int(q_lens.sum())
        cu = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu[1:])
        want_rows = [int(cu[i]) + int(p) for i, places in enumerate(want) for p in places]
        W = len(want_rows)
        tables = {gi: cache.page_table(gi, slots) for gi in cache.kv_groups}

        sizes = [T, T, T, n + 1, n, n, W] + [t.size for t in tables.values()]
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + _round4(s))
        if offs[-1] > self._host.numel():
            if self._event is not None:
                self._event.synchronize()
            self._grow(max(offs[-1], 2 * self._host.numel()))
        elif self._event is not None:
            self._event.synchronize()      # the last transfer has read the host buffer
        buf = self._np
        flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists]) if T else np.zeros(0, np.int64)
        seq_of = np.repeat(np.arange(n, dtype=np.int64), q_lens)
        pos = np.arange(T, dtype=np.int64) - cu[seq_of] + starts[seq_of]
        buf[offs[0]:offs[0] + T] = flat
        buf[offs[1]:offs[1] + T] = pos
        buf[offs[2]:offs[2] + T] = seq_of
        buf[offs[3]:offs[3] + n + 1] = cu
        buf[offs[4]:offs[4] + n] = np.asarray(slots, dtype=np.int64)
        buf[offs[5]:offs[5] + n] = starts + q_lens
        buf[offs[6]:offs[6] + W] = np.asarray(want_rows, dtype=np.int64)
        for k, t in enumerate(tables.values()):
            buf[offs[7 + k]:offs[7 + k] + t.size] = t.reshape(-1)
        total = offs[-1]
        self.last_h2d_bytes = 4 * total
        self._dev[:total].copy_(self._host[:total], non_blocking=True)
        if self.device.type == "cuda":
            self._event = torch.cuda.Event()
            self._event.record()
        d = self._dev

        def view(k: int, count: int) -> torch.Tensor:
            return d[offs[k]:offs[k] + count]

        ctx = StepContext(
            n_seqs=n, n_tokens=T, decode=bool((q_lens == 1).all()), max_q_len=int(q_lens.max()),
            max_kv_len=int((starts + q_lens).max()), page_size=cache.page_size,
            max_positions=cache.max_seq_tokens,
            tokens=view(0, T), positions=view(1, T), seq_of_token=view(2, T), cu_seqlens=view(3, n + 1),
            slots=view(4, n), kv_lens=view(5, n), want_rows=view(6, W),
            q_lens_host=q_lens, starts_host=np.asarray(starts, dtype=np.int64))
        for k, (gi, t) in enumerate(tables.items()):
            ctx.page_tables[gi] = view(7 + k, t.size).view(n, t.shape[1])
        return ctx
