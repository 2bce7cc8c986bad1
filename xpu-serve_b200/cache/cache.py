"""The cache: a slot per sequence, keys and values per layer call, fixed-size state beside them.

Layer calls are grouped by what they need (parts/base.py: KVNeed, StateNeed). Calls
that keep every key of the same geometry form one group with one page pool and one
page table; calls that keep a window form another, whose pages behind the window are
given back as a sequence grows; calls with a fixed-size state (the short convolution's
last kernel-1 inputs here, any recurrent state elsewhere) form groups that hold one
row per slot. Each group owns its storage. A slot's length is advanced only by
`end_step`, and `begin_step` changes nothing unless everything the step needs is
available (the reference leaves a failed step's state as it was,
src/backend/cpu_ref/cpu_backend.cpp:157-177).

Storage of a key/value call: [pages, 2 (keys, values), kv_heads, page_size, head_dim].
Storage of a state call:     [max_slots, *shape].
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import itertools

import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .pools import CacheError, CacheFull, IndexPool

PAGE_SIZE = 64


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


class KVGroup:
    def __init__(self, need: KVNeed, calls: List[Tuple[int, int]], n_pages: int, page_size: int, max_slots: int,
                 max_seq_pages: int, dtype: torch.dtype, device):
        """`calls`: the (layer call, index of the need in that call's declaration) pairs this group serves."""
        self.need = need
        self.calls = list(calls)
        self.page_size = page_size
        self.pages = IndexPool(n_pages, "page")
        self.max_seq_pages = max_seq_pages
        # logical page -> physical page, -1 where none is held
        self.table = np.full((max_slots, max_seq_pages), -1, dtype=np.int32)
        self.first_held = np.zeros(max_slots, dtype=np.int64)    # pages below it were given back
        self.end_held = np.zeros(max_slots, dtype=np.int64)      # pages from it on are not held yet
        self.version = 0      # grows whenever a row of `table` changes (a staged copy of the table is then stale)
        # one page more than the pool hands out: padding rows of a fixed-size batch write there
        self.dummy_page = n_pages
        self.storage: Dict[Tuple[int, int], torch.Tensor] = {
            c: torch.zeros((n_pages + 1, 2, need.kv_heads, page_size, need.head_dim),
                           dtype=dtype, device=device) for c in calls}

    def _first_needed_page(self, start: int) -> int:
        """The lowest page a query at position `start` or later can still see."""
        if self.need.window <= 0:
            return 0
        return max(0, start - self.need.window + 1) // self.page_size

    def pages_wanted(self, slot: int, new_len: int) -> int:
        return max(0, _ceil_div(new_len, self.page_size) - int(self.end_held[slot]))

    def reserve(self, slot: int, new_len: int) -> None:
        want = self.pages_wanted(slot, new_len)
        if want == 0:
            return
        end = int(self.end_held[slot])
        if end + want > self.max_seq_pages:
            raise CacheError(f"a sequence of {new_len} positions exceeds the cache's {self.max_seq_pages} pages a sequence")
        self.table[slot, end:end + want] = self.pages.take(want)
        self.end_held[slot] = end + want
        self.version += 1

    def trim(self, slot: int, length: int) -> None:
        first = min(self._first_needed_page(length), int(self.end_held[slot]))
        lo = int(self.first_held[slot])
        if first > lo:
            self.pages.give_back(int(p) for p in self.table[slot, lo:first])
            self.table[slot, lo:first] = -1
            self.first_held[slot] = first
            self.version += 1

    def unreserve(self, slot: int, length: int) -> None:
        """Gives back the pages held beyond those that `length` positions need (a step that reserved and then
        failed)."""
        keep = max(_ceil_div(length, self.page_size), int(self.first_held[slot]))
        end = int(self.end_held[slot])
        if end > keep:
            self.pages.give_back(int(p) for p in self.table[slot, keep:end])
            self.table[slot, keep:end] = -1
            self.end_held[slot] = keep
            self.version += 1

    def release(self, slot: int) -> None:
        lo, hi = int(self.first_held[slot]), int(self.end_held[slot])
        self.pages.give_back(int(p) for p in self.table[slot, lo:hi])
        self.table[slot, :] = -1
        self.first_held[slot] = 0
        self.end_held[slot] = 0
        self.version += 1


class StateGroup:
    def __init__(self, need: StateNeed, calls: List[Tuple[int, int]], max_slots: int, compute_dtype: torch.dtype, device):
        self.need = need
        self.calls = list(calls)
        dtype = torch.float32 if need.dtype == "float32" else compute_dtype
        # One row more than there are slots: the state of padding rows. The calls' tensors are pieces of one
        # allocation, each from a 256-byte boundary on, so that a batch's slots are zeroed with one launch for the
        # whole group instead of one a call.
        row = 1
        for n in need.shape:
            row *= int(n)
        item = torch.empty((), dtype=dtype).element_size()
        piece = -(-((max_slots + 1) * row * item) // 256) * 256 // item
        self._backing = torch.zeros(max(len(self.calls), 1) * piece, dtype=dtype, device=device)
        self._rows = self._backing.as_strided((len(self.calls), max_slots + 1, row), (piece, row, 1))
        self.storage: Dict[Tuple[int, int], torch.Tensor] = {
            c: self._backing[i * piece:i * piece + (max_slots + 1) * row].view(max_slots + 1, *need.shape)
            for i, c in enumerate(self.calls)}

    def zero(self, slots: torch.Tensor) -> None:
        if self.calls:
            self._rows.index_fill_(1, slots, 0)


@dataclass
class CallView:
    """What a mixer is handed for one layer call: the storage of its need. A mixer that declared several
    needs finds them in declaration order as `view[0]`, `view[1]`, ... (`view.storage` is then the first's)."""
    call: int
    group: int                 # index into Cache.groups; -1 for none
    storage: Optional[torch.Tensor]
    need: object
    owner: bool                # False when this call reads another call's cache
    parts: Tuple["CallView", ...] = ()

    def __getitem__(self, k: int) -> "CallView":
        return self.parts[k] if self.parts else (self,)[k]

    def __len__(self) -> int:
        return len(self.parts) if self.parts else (0 if self.storage is None else 1)


def _as_needs(need) -> Tuple[object, ...]:
    """A call's declaration as a tuple of needs: none, one, or several."""
    if need is None:
        return ()
    if isinstance(need, (tuple, list)):
        return tuple(need)
    return (need,)


_SERIALS = itertools.count(1)


class Cache:
    """needs[i] is what call i of the running order keeps per sequence (None: nothing; a KVNeed or a
    StateNeed; or a tuple of them), and shares[i] the call whose cache call i reads (None: its own)."""

    def __init__(self, needs: Sequence[object], shares: Sequence[Optional[int]], max_tokens: int, *,
                 page_size: int = PAGE_SIZE, max_slots: Optional[int] = None,
                 max_seq_tokens: Optional[int] = None, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.serial = next(_SERIALS)       # unlike id(), never given to another cache
        self.page_size = page_size
        self.max_tokens = _ceil_div(max_tokens, page_size) * page_size
        n_pages = self.max_tokens // page_size
        self.max_slots = n_pages if max_slots is None else max_slots
        self.max_seq_tokens = self.max_tokens if max_seq_tokens is None else min(max_seq_tokens, self.max_tokens)
        max_seq_pages = _ceil_div(self.max_seq_tokens, page_size)
        self.device = torch.device(device)
        self.dtype = dtype
        self.slots = IndexPool(self.max_slots, "slot")
        self.dummy_slot = self.max_slots      # never handed out; padding rows of a fixed-size batch use it
        self.lens = np.zeros(self.max_slots, dtype=np.int64)
        self.groups: List[object] = []
        needs = [_as_needs(n) for n in needs]
        # storage is keyed by (call, index of the need within the call's declaration)
        by_need: Dict[object, List[Tuple[int, int]]] = {}
        for call, (declared, share) in enumerate(zip(needs, shares)):
            if share is None:
                for k, need in enumerate(declared):
                    by_need.setdefault(need, []).append((call, k))
        self._group_of: Dict[Tuple[int, int], int] = {}
        for need, keys in by_need.items():
            if isinstance(need, KVNeed):
                g: object = KVGroup(need, keys, n_pages, page_size, self.max_slots, max_seq_pages, dtype, self.device)
            elif isinstance(need, StateNeed):
                g = StateGroup(need, keys, self.max_slots, dtype, self.device)
            else:
                raise TypeError(f"call {keys[0][0]} declares an unknown cache need {need!r}")
            for key in keys:
                self._group_of[key] = len(self.groups)
            self.groups.append(g)
        self.views: List[CallView] = []
        for call, (declared, share) in enumerate(zip(needs, shares)):
            src = call if share is None else share
            parts = []
            # a reader of another call's cache that declares no need of its own reads nothing
            for k in range(len(needs[src]) if (share is None or declared) else 0):
                gi = self._group_of[(src, k)]
                parts.append(CallView(call, gi, self.groups[gi].storage[(src, k)], self.groups[gi].need, share is None))
            if not parts:
                self.views.append(CallView(call, -1, None, None, True))
            elif len(parts) == 1:
                self.views.append(parts[0])
            else:
                first = parts[0]
                self.views.append(CallView(call, first.group, first.storage, first.need, first.owner, tuple(parts)))
        self.kv_groups = [i for i, g in enumerate(self.groups) if isinstance(g, KVGroup)]
        self._any_window = any(self.groups[i].need.window > 0 for i in self.kv_groups)
        self._last_slots: Optional[tuple] = None       # the batch of the last finished step (decode fast path)
        self._last_slots_arr: Optional[np.ndarray] = None

    # ------------------------------------------------------------ sequences
    def open(self, n: int) -> List[int]:
        """n free slots, their fixed-size state zeroed and their length 0."""
        slots = self.slots.take(n)
        self.lens[slots] = 0
        self._last_slots = None
        state_groups = [g for g in self.groups if isinstance(g, StateGroup)]
        if state_groups and slots:
            idx = torch.tensor(slots, dtype=torch.int64, device=self.device)
            for g in state_groups:
                g.zero(idx)
        return slots

    def close(self, slots: Sequence[int]) -> None:
        slots = list(slots)
        self._last_slots = None
        for s in slots:
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is freed twice or was never held")
        if len(set(slots)) != len(slots):
            raise CacheError("a slot is freed twice in one call")
        for s in slots:
            for g in self.groups:
                if isinstance(g, KVGroup):
                    g.release(s)
            self.lens[s] = 0
        self.slots.give_back(slots)

    # ---------------------------------------------------------------- steps
    def begin_step(self, slots: Sequence[int], q_lens: Sequence[int]) -> np.ndarray:
        """Reserves what the step writes. Returns each sequence's length before the step.
        Raises, with nothing changed, when a slot is not held, a sequence would outgrow
        max_seq_tokens, or pages run out."""
        if len(slots) != len(q_lens) or len(slots) == 0:
            raise CacheError("a step needs one token count per slot, and at least one slot")
        if self._same_decode_batch(slots, q_lens):
            # the batch of the last step again, one token each, no sequence at a page's or the context's end:
            # nothing to reserve, nothing that can fail
            return self.lens[self._last_slots_arr].copy()
        if len(set(slots)) != len(slots):
            raise CacheError("a slot appears twice in one step")
        for s, q in zip(slots, q_lens):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not held")
            if q <= 0:
                raise CacheError(f"slot {s}: a step needs at least one token")
            if self.lens[s] + q > self.max_seq_tokens:
                raise CacheError(f"slot {s}: {int(self.lens[s]) + q} positions exceed the limit of "
                                 f"{self.max_seq_tokens} a sequence")
        for gi in self.kv_groups:
            g = self.groups[gi]
            want = sum(g.pages_wanted(s, int(self.lens[s]) + q) for s, q in zip(slots, q_lens))
            if want > g.pages.free_count:
                raise CacheFull(f"the step needs {want} more pages, {g.pages.free_count} of {g.pages.count} are free")
        starts = self.lens[list(slots)].copy()
        for gi in self.kv_groups:
            g = self.groups[gi]
            for s, q in zip(slots, q_lens):
                g.reserve(s, int(self.lens[s]) + q)
        return starts

    def _same_decode_batch(self, slots: Sequence[int], q_lens: Sequence[int]) -> bool:
        """Whether this is the batch that `end_step` last saw, each sequence with one token that fits the pages
        it holds (so every check of `begin_step` would pass and no table would change)."""
        if self._last_slots is None or len(slots) != len(self._last_slots) or tuple(slots) != self._last_slots:
            return False
        if any(q != 1 for q in q_lens):
            return False
        lens = self.lens[self._last_slots_arr]
        if int(lens.max()) + 1 > self.max_seq_tokens or (lens % self.page_size == 0).any():
            return False
        return all(self.slots.is_held(s) for s in slots)

    def abort_step(self, slots: Sequence[int]) -> None:
        """Undoes `begin_step` for a step that failed before `end_step`: pages reserved for the step's tokens
        go back, lengths stay. The books are then as before the step. What the step's kernels had already
        written (fixed-size state, keys and values at the step's positions) is not undone: a sequence of a
        failed step cannot go on and has to be closed."""
        self._last_slots = None
        for s in slots:
            for gi in self.kv_groups:
                self.groups[gi].unreserve(s, int(self.lens[s]))

    def end_step(self, slots: Sequence[int], q_lens: Sequence[int]) -> None:
        key = tuple(slots)
        if key != self._last_slots:
            self._last_slots = key
            self._last_slots_arr = np.asarray(slots, dtype=np.int64)
        if not self._any_window and len(set(q_lens)) == 1:
            self.lens[self._last_slots_arr] += q_lens[0]
            return
        for s, q in zip(slots, q_lens):
            self.lens[s] += q
            for gi in self.kv_groups:
                g = self.groups[gi]
                if g.need.window > 0:
                    g.trim(s, int(self.lens[s]))

    def page_table(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> np.ndarray:
        """[len(slots), width] int32 rows of the group's table (width: the widest row held)."""
        g = self.groups[group]
        if width is None:
            width = max(1, int(g.end_held[list(slots)].max()))
        return g.table[list(slots), :width]

    def page_table_fixed(self, group: int, slots: Sequence[int], rows: int) -> np.ndarray:
        """[rows, max pages a sequence] int32: the slots' rows, then padding rows that name the
        group's spare page."""
        g = self.groups[group]
        out = np.full((rows, g.max_seq_pages), g.dummy_page, dtype=np.int32)
        out[:len(slots)] = g.table[list(slots)]
        return out

    def tables_version(self) -> int:
        """Changes whenever any key/value group's page table does."""
        return sum(self.groups[gi].version for gi in self.kv_groups)

    def tokens_held(self) -> int:
        """Positions reserved in the largest key/value group, in whole pages."""
        return max((self.groups[gi].pages.held_count for gi in self.kv_groups), default=0) * self.page_size

    def check(self) -> None:
        self.slots.check()
        for gi in self.kv_groups:
            g = self.groups[gi]
            g.pages.check()
            held = [int(p) for s in range(self.max_slots) for p in g.table[s] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError("a page is in two page tables")
            if len(held) != g.pages.held_count:
                raise CacheError(f"{g.pages.held_count} pages are held but the tables name {len(held)}")
            for s in range(self.max_slots):
                if not self.slots.is_held(s) and (g.table[s] >= 0).any():
                    raise CacheError(f"free slot {s} still has pages")
