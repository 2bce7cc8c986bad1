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
    want_all: bool = False       # want_rows is every row, in order
    page_tables: Dict[int, torch.Tensor] = field(default_factory=dict)
    q_lens_host: Optional[np.ndarray] = None
    starts_host: Optional[np.ndarray] = None
    fixed_shape: bool = False    # the step is (being captured as) a graph for any lengths up to max_q_len / max_kv_len:
                                 # parts choose their kernels and grids from those bounds, not from q_lens_host


class StepStager:
    """Owns the pinned host buffer and the device buffer that a step's description goes through."""

    def __init__(self, device, capacity: int = 1 << 16, fixed: bool = False):
        self.device = torch.device(device)
        self.fixed = fixed           # a captured graph holds this buffer's addresses: it must not be replaced
        self._host = None
        self._dev = None
        self._event = None
        self._fixed_layout = None     # set by stage_decode_fixed: what restage_next_token may rewrite
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
        want_rows = np.asarray([int(cu[i]) + int(p) for i, places in enumerate(want) for p in places], dtype=np.int64)
        tables = {gi: cache.page_table(gi, slots) for gi in cache.kv_groups}
        flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists]) if T else np.zeros(0, np.int64)
        seq_of = np.repeat(np.arange(n, dtype=np.int64), q_lens)
        pos = np.arange(T, dtype=np.int64) - cu[seq_of] + starts[seq_of]
        return self._emit(cache, flat, pos, seq_of, cu, np.asarray(slots, dtype=np.int64), starts + q_lens, want_rows,
                          tables, q_lens, np.asarray(starts, dtype=np.int64), int((starts + q_lens).max()))

    def stage_decode_fixed(self, cache, slots: Sequence[int], tokens: Sequence[int], starts: np.ndarray,
                           rows: int, kv_limit: Optional[int] = None) -> StepContext:
        """One token for each of `slots`, laid out as a batch of exactly `rows` sequences with page
        tables of the cache's full width, so that the layout (and every address a captured graph
        reads) is the same from step to step. Rows past len(slots) are padding: they use the cache's
        spare slot and page, stand at position 0 and are never read by the real rows. `kv_limit`: the most keys
        a sequence of this step will have (what the launches that are captured size their key splits by);
        the cache's own limit when not given."""
        n = len(slots)
        tok = np.zeros(rows, dtype=np.int64)
        tok[:n] = np.asarray(tokens, dtype=np.int64)
        pos = np.zeros(rows, dtype=np.int64)
        pos[:n] = starts
        sl = np.full(rows, cache.dummy_slot, dtype=np.int64)
        sl[:n] = np.asarray(slots, dtype=np.int64)
        idx = np.arange(rows, dtype=np.int64)
        tables = {gi: cache.page_table_fixed(gi, slots, rows) for gi in cache.kv_groups}
        q_lens = np.ones(rows, dtype=np.int64)
        ctx = self._emit(cache, tok, pos, idx, np.arange(rows + 1, dtype=np.int64), sl, pos + 1, idx, tables, q_lens,
                         pos, cache.max_seq_tokens if kv_limit is None else min(kv_limit, cache.max_seq_tokens))
        r4 = _round4(rows)
        # (sequences, offsets of tokens, positions and lengths, words up to the end of the lengths)
        self._fixed_layout = (n, 0, r4, 3 * r4 + _round4(rows + 1) + r4, 3 * r4 + _round4(rows + 1) + 2 * r4)
        return ctx

    def stage_prompt_fixed(self, cache, slot: int, tokens: Sequence[int], start: int, rows: int) -> StepContext:
        """One sequence's next `len(tokens)` tokens (at most `rows`), laid out as a step of exactly `rows` tokens in
        two sequences: the real one, then a padding sequence of the remaining rows (none when the piece fills the step)
        in the cache's spare slot and page (nothing it computes is ever read). The layout, every address and every
        size that a kernel launch gets from the host depend on `rows` and the cache alone, so a graph captured for `rows` serves any shorter prompt piece at any
        position. The logits wanted are the real sequence's last row's."""
        T = len(tokens)
        if not 0 < T <= rows:
            raise ValueError(f"{T} tokens do not fit a fixed step of {rows} rows")
        tok = np.zeros(rows, dtype=np.int64)
        tok[:T] = np.asarray(tokens, dtype=np.int64)
        pos = np.concatenate([np.arange(start, start + T, dtype=np.int64), np.arange(rows - T, dtype=np.int64)])
        seq_of = np.concatenate([np.zeros(T, dtype=np.int64), np.ones(rows - T, dtype=np.int64)])
        cu = np.asarray([0, T, rows], dtype=np.int64)
        sl = np.asarray([slot, cache.dummy_slot], dtype=np.int64)
        kv = np.asarray([start + T, rows - T], dtype=np.int64)
        real = [] if slot == cache.dummy_slot else [slot]        # (a capture runs in the spare slot: spare pages for both rows)
        tables = {gi: cache.page_table_fixed(gi, real, 2) for gi in cache.kv_groups}
        ctx = self._emit(cache, tok, pos, seq_of, cu, sl, kv, np.asarray([T - 1], dtype=np.int64), tables,
                         np.asarray([rows, rows], dtype=np.int64), np.asarray([start, 0], dtype=np.int64), cache.max_seq_tokens)
        ctx.decode, ctx.max_q_len, ctx.fixed_shape, ctx.want_all = False, rows, True, False
        return ctx

    def restage_next_token(self, tokens: Sequence[int], starts: np.ndarray) -> bool:
        """The step after a `stage_decode_fixed` of the same sequences, whose page tables have not changed:
        only the tokens, the positions and the lengths differ, so only those are rewritten and copied.
        False (nothing done) when the last staging was not such a step or the positions do not follow on."""
        lay = self._fixed_layout
        n = len(tokens)
        if lay is None or n != lay[0]:
            return False
        _, o_tok, o_pos, o_kv, head = lay
        buf = self._np
        if not np.array_equal(buf[o_pos:o_pos + n] + 1, starts):
            return False
        if self._event is not None:
            self._event.synchronize()
        buf[o_tok:o_tok + n] = tokens
        buf[o_pos:o_pos + n] += 1
        buf[o_kv:o_kv + n] += 1
        self.last_h2d_bytes = 4 * head
        self._dev[:head].copy_(self._host[:head], non_blocking=True)
        self._event.record()
        return True

    def feed_tokens(self, tokens_dev: torch.Tensor, n: int) -> None:
        """The first n tokens of the staged step are taken from a device tensor (int32) instead of the host's."""
        self._dev[:n].copy_(tokens_dev[:n])

    def restage_fed(self, tokens_dev: torch.Tensor, n: int, starts: np.ndarray) -> bool:
        """`restage_next_token` with the tokens coming from the device: positions and lengths advance on the
        host and are copied; the tokens never leave the device."""
        lay = self._fixed_layout
        if lay is None or n != lay[0]:
            return False
        _, o_tok, o_pos, o_kv, head = lay
        buf = self._np
        if not np.array_equal(buf[o_pos:o_pos + n] + 1, starts):
            return False
        if self._event is not None:
            self._event.synchronize()
        buf[o_pos:o_pos + n] += 1
        buf[o_kv:o_kv + n] += 1
        self.last_h2d_bytes = 4 * (head - o_pos)
        self._dev[o_pos:head].copy_(self._host[o_pos:head], non_blocking=True)
        self._event.record()
        self.feed_tokens(tokens_dev, n)
        return True

    def _emit(self, cache, flat, pos, seq_of, cu, slots, kv_lens, want_rows, tables, q_lens, starts,
              max_kv_len) -> StepContext:
        T, n, W = len(flat), len(slots), len(want_rows)
        self._fixed_layout = None
        sizes = [T, T, T, n + 1, n, n, W] + [t.size for t in tables.values()]
        offs = [0]
        for sz in sizes:
            offs.append(offs[-1] + _round4(sz))
        if self._event is not None:
            self._event.synchronize()      # the last transfer has read the host buffer
        if offs[-1] > self._host.numel():
            if self.fixed:
                raise RuntimeError("a step's description outgrew a buffer whose addresses a graph holds")
            self._grow(max(offs[-1], 2 * self._host.numel()))
        buf = self._np
        for k, a in enumerate((flat, pos, seq_of, cu, slots, kv_lens, want_rows)):
            buf[offs[k]:offs[k] + len(a)] = a
        for k, t in enumerate(tables.values()):
            buf[offs[7 + k]:offs[7 + k] + t.size] = t.reshape(-1)
        total = offs[-1]
        self.last_h2d_bytes = 4 * total
        self._dev[:total].copy_(self._host[:total], non_blocking=True)
        if self.device.type == "cuda":
            if self._event is None:
                self._event = torch.cuda.Event()
            self._event.record()
        d = self._dev

        def view(k: int, count: int) -> torch.Tensor:
            return d[offs[k]:offs[k] + count]

        ctx = StepContext(
            n_seqs=n, n_tokens=T, decode=bool((q_lens == 1).all()), max_q_len=int(q_lens.max()),
            max_kv_len=int(max_kv_len), page_size=cache.page_size, max_positions=cache.max_seq_tokens,
            tokens=view(0, T), positions=view(1, T), seq_of_token=view(2, T), cu_seqlens=view(3, n + 1),
            slots=view(4, n), kv_lens=view(5, n), want_rows=view(6, W),
            want_all=bool(W == T and np.array_equal(np.asarray(want_rows, dtype=np.int64), np.arange(T, dtype=np.int64))),
            q_lens_host=q_lens, starts_host=starts)
        for k, (gi, t) in enumerate(tables.items()):
            ctx.page_tables[gi] = view(7 + k, t.size).view(n, t.shape[1])
        return ctx
