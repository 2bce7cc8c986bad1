"""The Python entry point: a model folder in, tokens out.

    engine = Engine(model_dir, precision="bf16", ctx=4096)
    results = engine.generate([GenerateRequest(prompt=[1, 2, 3], max_new_tokens=16)])

The reference's entry is `EngineService::create(model_dir, options)` and
`generate(request, on_token)` (src/service/engine_service.cpp:30-124,
src/engine/engine.h:40); the option names `precision`, `ctx` and `prefill_chunk` are its
command line's (src/cli/main.cpp:72-125). `ctx` is clamped to the model's
max_position_embeddings as there (engine_service.cpp:54-58). Batching is added: `generate`
takes a list of requests and returns their results in the same order.
"""
from __future__ import annotations

import os
import secrets
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import lib as ops
from ..sampling.params import (GenerateRequest, GenerateResult, SamplingParams, TokenCallback, merged_stop_ids,
                               read_generation_defaults)
from .generate import generate as _generate
from .model import Model, load_model

PRECISIONS = {"bf16": "bfloat16", "bfloat16": "bfloat16", "f32": "float32", "float32": "float32"}


def _i64(v: int) -> int:
    """A 64-bit seed as the signed value with the same bits (torch has no unsigned 64-bit tensors)."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


class _Handle:
    __slots__ = ("slot", "row", "request", "seed", "counter")

    def __init__(self, slot, row, request, seed):
        self.slot, self.row, self.request, self.seed, self.counter = slot, row, request, seed, 0


class _Ahead:
    """A decode step that was started before the loop asked for it. `chosen`: its tokens on the device."""
    __slots__ = ("row_of", "fed", "event", "host", "chosen", "status_at")

    def __init__(self, row_of, fed, event, host, chosen, status_at=None):
        self.row_of, self.fed, self.event, self.host, self.chosen = row_of, fed, event, host, chosen
        self.status_at = status_at       # where in `host` the status word of kernels with bounded waits lies, if it travels


class _Choice:
    """What the sampling kernels need for one set of sequences, on the device for as long as the same sequences
    are chosen for step after step: the parameters do not change, and the draw counters advance by one a step,
    on the device too. `counters_host` mirrors them so that a step that does not follow on is noticed."""

    def __init__(self, chosen: Sequence[_Handle], device, with_penalties: bool, offset: int):
        params = [h.request.sampling for h in chosen]
        f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=device)          # noqa: E731
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)            # noqa: E731
        self.key = tuple(chosen)
        self.all_greedy = all(p.greedy() for p in params)
        if not self.all_greedy:
            self.temperature, self.top_k = f32([p.temperature for p in params]), i32([p.top_k for p in params])
            self.top_p, self.min_p = f32([p.top_p for p in params]), f32([p.min_p for p in params])
            self.seeds = torch.tensor([_i64(h.seed) for h in chosen], dtype=torch.int64, device=device)
        self.counters_host = [h.counter + offset for h in chosen]
        if not self.all_greedy:
            self.counters = torch.tensor(self.counters_host, dtype=torch.int64, device=device)
        if with_penalties:
            self.rows = i32([h.row for h in chosen])
            self.repetition = f32([p.repetition_penalty for p in params])
            self.presence = f32([p.presence_penalty for p in params])
            self.frequency = f32([p.frequency_penalty for p in params])


class DeviceStepper:
    """Runs the generation loop's steps on the device: the model's step function, then the choice of
    the next token by the sampling kernels; only token ids cross to the host.

    Running ahead. A generation loop feeds every live sequence the token the last step chose for it, so
    while sequences decode, the step after the one being asked for is started at once, fed on the device
    from the graph's own argmax (greedy sequences) or from what the sampling kernels chose (seeded draws,
    penalties; the draw for the step that runs ahead uses the sequence's next counter); by the time the loop
    has looked at a step's tokens the next step is already running. A sequence that the loop ends (a stop
    token, its length, a callback) has then run one step too many: a row of work that nobody reads, in a
    slot that the loop closes. The promise the loop
    makes in return (`generate` keeps it): after decoding has begun, a sequence's next call brings the token
    the last call returned for it. A call that breaks it is refused."""

    def __init__(self, model: Model, max_tokens: int, max_context: int, max_slots: Optional[int] = None):
        self.model = model
        self.cache = model.new_cache(max_tokens, max_slots=max_slots, max_seq_tokens=max_context)
        self.max_context = self.cache.max_seq_tokens
        self.capacity_tokens = self.cache.max_tokens
        self.page_size = self.cache.page_size
        self.max_slots = self.cache.max_slots
        self.device = model.rt.device
        self._pen = None        # (seen uint8 [rows, V], counts int32 [rows, V]) when a batch has penalties
        self._rows_free: List[int] = []
        self._host_bufs: List[torch.Tensor] = []              # pinned: where the chosen tokens land, in turns
        self._turn = 0
        self.run_ahead = os.environ.get("XS_NO_RUN_AHEAD", "0") != "1"
        self._ahead: Optional[_Ahead] = None
        self._choice: Optional[_Choice] = None
        self._live = set()          # handles that hold a slot
        self._out_bufs: List[Optional[torch.Tensor]] = [None, None]      # where the sampling kernels leave their choice
        self._out_turn = 0

    # ---------------------------------------------------------------- slots
    def open(self, requests: Sequence[GenerateRequest]) -> List[_Handle]:
        self._ahead = None          # what ran ahead for an earlier batch is nobody's any more
        self._choice = None
        slots = self.cache.open(len(requests))
        handles = []
        for row, (s, r) in enumerate(zip(slots, requests)):
            seed = r.sampling.seed if r.sampling.seed is not None else secrets.randbits(63)
            handles.append(_Handle(s, row, r, seed))
        self._live.update(handles)
        if any(r.sampling.has_penalties() for r in requests):
            V = self.model.spec.vocab
            seen = torch.zeros((len(requests), V), dtype=torch.uint8, device=self.device)
            counts = torch.zeros((len(requests), V), dtype=torch.int32, device=self.device)
            toks = torch.tensor([t for r in requests for t in r.prompt], dtype=torch.int32, device=self.device)
            rows = torch.tensor([i for i, r in enumerate(requests) for _ in r.prompt], dtype=torch.int32,
                                device=self.device)
            ops.note_tokens(toks, rows, seen, counts, generated=False)
            self._pen = (seen, counts)
        else:
            self._pen = None
        return handles

    def close(self, handles: Sequence[_Handle]) -> None:
        self.cache.close([h.slot for h in handles])
        self._live.difference_update(handles)

    # ----------------------------------------------------------------- step
    def step(self, handles: Sequence[_Handle], token_lists, want: Sequence[bool]) -> List[Optional[int]]:
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            if any(h in ahead.row_of for h in handles):
                return self._take_ahead(ahead, handles, token_lists, want)
            if any(h in self._live for h in ahead.row_of):
                raise RuntimeError("this stepper runs one decode step ahead for sequences that are still open; "
                                   "their step has to be taken before other sequences are stepped")
        places = [[len(t) - 1] if w else [] for t, w in zip(token_lists, want)]
        logits = self.model.step(self.cache, [h.slot for h in handles], token_lists, places)
        chosen = [h for h, w in zip(handles, want) if w]
        if not chosen:
            return [None] * len(handles)
        n = len(chosen)
        dev = self.device
        params = [h.request.sampling for h in chosen]
        if self._pen is None and n == len(handles) and self.model.last_greedy is not None and all(p.greedy() for p in params):
            # the decode graph has chosen already; start the next step before waiting for this one's tokens
            host, event, status_at = self._copy_out(self.model.last_greedy)
            self._start_ahead(handles)
            self._landed(host, event, status_at)
            tokens = host[:n].tolist()
            if self._ahead is not None:
                self._ahead.fed = tokens
            for h in chosen:
                h.counter += 1
            return tokens
        out = self._choose(logits, chosen, 0)
        host, event, status_at = self._copy_out(out)
        if n == len(handles):
            self._start_ahead(handles, out)       # the next step, fed on the device, before waiting for this one
        self._landed(host, event, status_at)
        tokens = host[:n].tolist()
        for h in chosen:
            h.counter += 1
        if self._ahead is not None:
            self._ahead.fed = tokens
        if n == len(want):
            return tokens
        it = iter(tokens)
        return [next(it) if w else None for w in want]

    def _choose(self, logits: torch.Tensor, chosen: Sequence[_Handle], offset: int) -> torch.Tensor:
        """The sampling kernels over `logits` (one row per chosen sequence): penalties, then argmax or a seeded
        draw with each sequence's draw counter (+ offset: 1 for a step that runs ahead of the loop's count), then
        the note of the chosen tokens for the penalties. Returns the tokens, int32 on the device."""
        c = self._choice
        expected = [h.counter + offset for h in chosen]
        if c is None or c.key != tuple(chosen) or c.counters_host != expected:
            c = self._choice = _Choice(chosen, self.device, self._pen is not None, offset)
        self._out_turn ^= 1                    # two buffers in turns: a step that runs ahead chooses while the last
        out = self._out_bufs[self._out_turn]   # step's choice is still on its way to the host
        if out is None or out.numel() < len(chosen):
            out = self._out_bufs[self._out_turn] = torch.empty(max(64, 2 * len(chosen)), dtype=torch.int32, device=self.device)
        out = out[:len(chosen)]
        if self._pen is not None:
            ops.apply_penalties(logits, self._pen[0], self._pen[1], c.rows, c.repetition, c.presence, c.frequency)
        if c.all_greedy:
            ops.argmax(logits, out)           # (no draw: the device's counters are not used, the host's mirror goes on)
        else:
            ops.sample(logits, c.temperature, c.top_k, c.top_p, c.min_p, c.seeds, c.counters, out, advance=True)
        c.counters_host = [v + 1 for v in c.counters_host]
        if self._pen is not None:
            ops.note_tokens(out, c.rows, self._pen[0], self._pen[1], generated=True)
        return out

    def _copy_out(self, out: torch.Tensor):
        """Starts the step's only device-to-host copy (the chosen tokens, into pinned memory) and returns the
        host buffer, the event that says it has landed and where in the buffer a status word lies (None:
        nowhere). Two buffers take turns: a step that runs ahead copies out while the one before it is still
        being read. When a kernel with bounded waits ran since the
        status word was last read (the tcgen05 kernels of prompt steps; decode attention at head size 64), the
        word travels behind the tokens and `_landed` looks at it."""
        n = out.numel()
        self._turn ^= 1
        while len(self._host_bufs) < 2:
            self._host_bufs.append(torch.empty(64, dtype=torch.int32, pin_memory=True))
        if self._host_bufs[self._turn].numel() < n + 1:
            self._host_bufs[self._turn] = torch.empty(2 * n + 1, dtype=torch.int32, pin_memory=True)
        host = self._host_bufs[self._turn]
        host[:n].copy_(out, non_blocking=True)
        status_at = None
        if ops.tc_status_unread(self.device):
            host[n:n + 1].copy_(ops.gemm_tc_status(self.device), non_blocking=True)
            status_at = n
        event = torch.cuda.Event()
        event.record()
        return host, event, status_at

    def _landed(self, host: torch.Tensor, event, status_at: Optional[int]) -> None:
        """Waits for a `_copy_out`, and fails the step if the status word that came with it is set."""
        event.synchronize()
        if status_at is not None:
            ops.tc_status_read(int(host[status_at]), self.device)

    # ----------------------------------------------------------- running ahead
    def _start_ahead(self, handles: Sequence[_Handle], chosen_dev: Optional[torch.Tensor] = None) -> None:
        """Starts the decode step after the last one for the same sequences, fed on the device, if the last
        step was a graph step of exactly these sequences and the cache has room. Greedy sequences without
        penalties are fed the graph's own argmax; the others `chosen_dev`, what the sampling kernels chose from
        the last step's logits, and their next tokens are chosen at once too."""
        if not self.run_ahead:
            return
        slots = [h.slot for h in handles]
        if self._pen is None and all(h.request.sampling.greedy() for h in handles):
            out = self.model.step_from_last_greedy(self.cache, slots)
        else:
            if chosen_dev is None:
                return
            logits = self.model.step_fed(self.cache, slots, chosen_dev)
            out = None if logits is None else self._choose(logits, handles, 1)
        if out is None:
            return
        host, event, status_at = self._copy_out(out)
        self._ahead = _Ahead({h: i for i, h in enumerate(handles)}, None, event, host, out, status_at)

    def _take_ahead(self, ahead: _Ahead, handles, token_lists, want) -> List[Optional[int]]:
        """The loop now asks for (a part of) the step that already runs."""
        for h, toks, w in zip(handles, token_lists, want):
            i = ahead.row_of.get(h)
            if i is None or not w or len(toks) != 1 or int(toks[0]) != ahead.fed[i]:
                raise RuntimeError("this stepper runs one decode step ahead: after decoding has begun, a sequence's "
                                   "next step must bring the token that the last step returned for it")
        if len(handles) == len(ahead.row_of) and [ahead.row_of[h] for h in handles] == list(range(len(handles))):
            self._start_ahead(handles, ahead.chosen)          # the same sequences go on: keep the device busy
        self._landed(ahead.host, ahead.event, ahead.status_at)
        tokens = ahead.host[:len(ahead.row_of)].tolist()
        got = [tokens[ahead.row_of[h]] for h in handles]
        if self._ahead is not None:
            self._ahead.fed = got
        for h in handles:
            h.counter += 1
        return got


class Engine:
    def __init__(self, model_dir: str, precision: str = "bf16", ctx: int = 8192, max_tokens: Optional[int] = None,
                 max_batch: int = 64, prefill_chunk: int = 8192, device: str = "cuda:0"):
        if precision not in PRECISIONS:
            raise ValueError(f"precision '{precision}' is not supported (bf16, f32 are)")
        self.model: Model = load_model(model_dir, dtype=PRECISIONS[precision], device=device)
        self.default_sampling, _ = read_generation_defaults(model_dir)
        self.stop_token_ids: List[int] = merged_stop_ids(model_dir, self.model.config)
        ctx = min(ctx, self.model.spec.max_position)
        self.max_batch = max_batch
        self.prefill_chunk = prefill_chunk
        if max_tokens is None:
            max_tokens = ctx * min(max_batch, 8)
        self.stepper = DeviceStepper(self.model, max_tokens, ctx, max_slots=max(max_batch, 1))

    @property
    def ctx(self) -> int:
        return self.stepper.max_context

    def generate(self, requests: Sequence[GenerateRequest], on_token: Optional[TokenCallback] = None
                 ) -> List[GenerateResult]:
        return _generate(self.stepper, requests, on_token, max_batch=self.max_batch,
                         prefill_chunk=self.prefill_chunk)

    def generate_tokens(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 32,
                        sampling: Optional[SamplingParams] = None, stop_token_ids: Optional[Sequence[int]] = None
                        ) -> List[List[int]]:
        """Token ids in, token ids out: one list of generated tokens per prompt."""
        sampling = sampling or self.default_sampling
        stops = list(self.stop_token_ids if stop_token_ids is None else stop_token_ids)
        reqs = [GenerateRequest(list(p), sampling, max_new_tokens, stops) for p in prompts]
        out = self.generate(reqs)
        for r in out:
            if r.finish == "error":
                raise RuntimeError(r.error)
        return [r.tokens for r in out]
