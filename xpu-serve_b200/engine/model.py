"""A model on a device: its parts, its cache, and the step function.

`Model.step` is the one function through which every token passes, for prompts and for
decoding, for generation and for trace replay. It takes a batch of sequences (their slots,
each one's next tokens, and the places whose logits are wanted), runs only those tokens
from what the cache holds, and returns float32 logits for the wanted places.

The reference runs one graph for one sequence per step (src/backend/backend.h:46-87,
src/models/lfm3/lfm3_model.cpp:34-44); the layer order and formulas are the same
(src/models/lfm3/lfm3_decoder.cpp:49-90), batching and the wanted places are added.
"""
from __future__ import annotations

import gc
import os
import weakref
from contextlib import contextmanager
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import registry
from ..cache import Cache, CacheError
from ..config.json_util import ConfigError, read_json
from ..config.spec import ModelSpec
from ..ops import lib as ops
from ..parts.block import ResidualStream
from ..weights.loader import load_weights
from .runtime import Runtime, Workspace
from .step import StepContext, StepStager


PROMPT_BUCKETS = (32, 64, 128, 256, 512)
MAX_DECODE_GRAPHS = 24      # per cache: (rows, bound on keys) pairs kept at one time


def _prompt_bucket(n: int) -> Optional[int]:
    """Rows of the graph that serves one sequence's piece of n tokens (the piece and its padding rows, if any), or None."""
    for b in PROMPT_BUCKETS:
        if n <= b:
            return b
    return None


def _bucket(n: int) -> int:
    """Batch sizes that decode graphs are captured for: exact up to 8, then multiples of 8 up to 64,
    then multiples of 32."""
    if n <= 8:
        return n
    if n <= 64:
        return -(-n // 8) * 8
    return -(-n // 32) * 32


def _kv_bucket(n: int, limit: int) -> int:
    """Key lengths that decode graphs are captured for: 1,024, 1,536, 2,048, 3,072, ... up to the cache's limit
    for one sequence. The split of a sequence's keys over CTAs is fixed when a graph is captured, so it should fit
    the lengths that the graph then sees: measured on B200 (1.2B shape, 2,048 cached tokens), a graph sized for
    131,072 keys takes 0.86 instead of 0.75 ms a step at batch 8 and 1.32 instead of 1.16 at batch 64."""
    b = 1024
    while b < n:
        b = b * 3 // 2 if (b & (b - 1)) == 0 else (b // 3) * 4
    return min(b, limit)


class _DecodeGraph:
    """A captured decode step for a fixed number of rows: its own scratch buffers and its own
    description buffer, whose addresses the graph holds."""

    def __init__(self, rows: int, graph, stager: StepStager, ws: Workspace, logits: torch.Tensor, greedy: torch.Tensor,
                 kernels: int, bounded: bool, kv_limit: Optional[int] = None):
        self.rows, self.graph, self.stager, self.ws, self.logits, self.kernels = rows, graph, stager, ws, logits, kernels
        self.kv_limit = kv_limit   # decode graphs: the most keys a sequence may have when this graph is replayed
        self.last_use = 0
        self.bounded = bounded     # the graph holds a kernel with bounded waits: its status word wants a look after a replay
        self.greedy = greedy       # int32 [rows]: each row's most likely token, found inside the graph
        self.batch_key = None      # (slots, version of the cache's page tables) of the step staged last


class Model:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], dtype: str = "bfloat16",
                 device="cuda:0", config=None):
        """`weights`: tensors by name without the model prefix (weights.loader.load_weights)."""
        spec.validate()
        self.spec, self.config = spec, config
        self.rt = Runtime(dtype, device)
        rt = self.rt
        self.embed = rt.matrix(weights[spec.names["embed"]])
        self.head = self.embed if spec.tied_head else rt.matrix(weights[spec.names["head"]])
        self.final_norm = registry.norm_class(spec.final_norm.kind)(spec.final_norm, weights, spec.names["final_norm"], rt)
        self.blocks: List[object] = []
        for layer in spec.layers:
            own = {k[len(layer.prefix):]: v for k, v in weights.items() if k.startswith(layer.prefix)}
            self.blocks.append(registry.arrangement_class(layer.kind)(layer, own, rt))
        self.stager = StepStager(rt.device)
        # Decode steps are launch-bound (some 150 small kernels): they are captured once per batch
        # size into a CUDA graph and replayed. XS_NO_GRAPHS=1 runs every step kernel by kernel.
        # (XS_PROFILE=1 and XS_SYNC=1, the per-launch timing and error-naming switches of ops/lib.py, do the same.)
        self.use_graphs = os.environ.get("XS_NO_GRAPHS", "0") != "1" and not ops.watched()
        self.last_greedy: Optional[torch.Tensor] = None
        self._last_graph: Optional[_DecodeGraph] = None
        # Decode graphs per cache (a graph holds the addresses of the cache's storage; by the cache's serial number,
        # which unlike its id() no later cache gets) and number of rows. When a cache is gone its graphs are set
        # aside and destroyed at the next decode step: the garbage collector may notice the cache in the middle
        # of a graph capture, where destroying a graph is not allowed.
        self._graphs: Dict[int, Dict[Tuple[int, int], _DecodeGraph]] = {}
        self._cache_refs: Dict[int, weakref.ref] = {}
        self._retired: List[Dict] = []
        self._uses = 0
        # Prompt steps of one sequence are bound by the host (some 130 launches at 10 to 15 us each, against half a
        # millisecond of device time for 128 tokens), so they are captured too: per cache and per number of rows (32 to
        # 512; the piece is padded with a sequence in the cache's spare slot). XS_NO_PROMPT_GRAPHS=1: kernel by kernel.
        # Only when every part of the model says that its prompt code can be captured for any lengths (parts/base.py).
        parts_ok = all(getattr(c, "fixed_shape_ok", False) for layer in spec.layers for c in (
            registry.arrangement_class(layer.kind), registry.mixer_class(layer.mixer.kind),
            registry.ffn_class(layer.ffn.kind), registry.norm_class(layer.norm.kind)))
        parts_ok = parts_ok and getattr(registry.norm_class(spec.final_norm.kind), "fixed_shape_ok", False)
        self.use_prompt_graphs = self.use_graphs and parts_ok and os.environ.get("XS_NO_PROMPT_GRAPHS", "0") != "1"
        self._prompt_graphs: Dict[int, Dict[int, _DecodeGraph]] = {}
        self.last_h2d_bytes = 0      # bytes of the last step's description copied to the device

    # ----------------------------------------------------------------- cache
    def cache_needs(self):
        needs, shares = [], []
        for call in self.spec.order:
            layer = self.spec.layers[call.layer]
            needs.append(registry.arrangement_class(layer.kind).cache_need(layer))
            shares.append(call.cache_of)
        return needs, shares

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None,
                  max_seq_tokens: Optional[int] = None) -> Cache:
        needs, shares = self.cache_needs()
        limit = self.spec.max_position if max_seq_tokens is None else min(max_seq_tokens, self.spec.max_position)
        return Cache(needs, shares, max_tokens, max_slots=max_slots, max_seq_tokens=limit,
                     dtype=self.rt.act_dtype, device=self.rt.device)

    # ------------------------------------------------------------------ step
    def check_tokens(self, token_lists: Sequence[Sequence[int]]) -> None:
        V = self.spec.vocab
        for toks in token_lists:
            for t in toks:
                if not 0 <= int(t) < V:
                    raise ValueError(f"token id {int(t)} outside the vocabulary ({V})")

    def step(self, cache: Cache, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Runs each sequence's next tokens. `want[i]` lists the places among sequence i's tokens of
        this step whose logits are returned (default: the last). Returns [wanted, vocab] float32 on
        the device, in the order of the sequences and of `want`. On an error the cache's books (lengths,
        pages held) are as before the step; a kernel that failed in the middle may already have written
        state, keys and values for the step's positions, so its sequences cannot go on and must be closed
        (the generation loop and trace replay do that)."""
        if want is None:
            want = [[len(t) - 1] for t in token_lists]
        if len(slots) != len(token_lists) or len(want) != len(slots):
            raise ValueError("a step needs one token list and one list of wanted places per slot")
        self.check_tokens(token_lists)
        for toks, places in zip(token_lists, want):
            for p in places:
                if not 0 <= int(p) < len(toks):
                    raise ValueError(f"wanted place {p} is not among the {len(toks)} tokens of the step")
        q_lens = [len(t) for t in token_lists]
        self.last_greedy = None      # set by a decode graph: argmax of the returned rows, already on the device
        self._last_graph = None
        starts = cache.begin_step(slots, q_lens)
        try:
            if self.use_graphs and max(q_lens) == 1:
                logits = self._decode_with_graph(cache, slots, token_lists, want, starts)
            elif (self.use_prompt_graphs and len(slots) == 1 and _prompt_bucket(q_lens[0]) is not None
                  and list(want[0]) == [q_lens[0] - 1]):
                logits = self._prompt_with_graph(cache, slots[0], token_lists[0], int(starts[0]))
            else:
                ctx = self.stager.stage(cache, slots, token_lists, want, starts)
                self.last_h2d_bytes = self.stager.last_h2d_bytes
                logits = self.forward(ctx, cache)
        except Exception:
            cache.abort_step(slots)
            raise
        cache.end_step(slots, q_lens)
        return logits

    # ---------------------------------------------------------- decode graphs
    @contextmanager
    def _workspace(self, ws: Workspace):
        old, self.rt.ws = self.rt.ws, ws
        try:
            yield
        finally:
            self.rt.ws = old

    def _graphs_of(self, cache: Cache) -> Dict[Tuple[int, int], _DecodeGraph]:
        self._retired.clear()            # no capture is under way here
        per_cache = self._graphs.get(cache.serial)
        if per_cache is None:
            per_cache = self._graphs[cache.serial] = {}
            serial, me = cache.serial, weakref.ref(self)

            def gone(_ref):
                model = me()
                if model is not None:
                    model._cache_refs.pop(serial, None)
                    for table in (model._graphs, model._prompt_graphs):
                        dead = table.pop(serial, None)
                        if dead:
                            model._retired.append(dead)

            self._cache_refs[serial] = weakref.ref(cache, gone)
        return per_cache

    def _decode_graph(self, cache: Cache, rows: int, keys: int) -> _DecodeGraph:
        """The graph for `rows` sequences of at most `keys` keys each, captured at its first use."""
        per_cache = self._graphs_of(cache)
        key = (rows, _kv_bucket(keys, cache.max_seq_tokens))
        g = per_cache.get(key)
        if g is None:
            g = per_cache[key] = self._capture(cache, rows, key[1])
            cache._graph_owner = self        # graphs die with the model; the cache only marks its use
            if len(per_cache) > MAX_DECODE_GRAPHS:       # each holds its scratch buffers and its logits: let the one unused longest go
                oldest = min((k for k in per_cache if k != key), key=lambda k: per_cache[k].last_use)
                self._retired.append({oldest: per_cache.pop(oldest)})    # destroyed at the next step, outside any capture
        self._uses += 1
        g.last_use = self._uses
        return g

    def _capture(self, cache: Cache, rows: int, kv_limit: int) -> _DecodeGraph:
        """Captures the decode step for `rows` sequences of at most `kv_limit` keys. Warm-up and capture run on
        padding rows only (the cache's spare slot and page), so no sequence's state is touched before the first replay."""
        rt = self.rt
        ws = Workspace(rt.device)
        width = sum(cache.groups[gi].max_seq_pages for gi in cache.kv_groups)
        stager = StepStager(rt.device, capacity=8 * rows + rows * width + 64, fixed=True)
        ctx = stager.stage_decode_fixed(cache, [], [], np.zeros(0, dtype=np.int64), rows, kv_limit)
        greedy = torch.empty(rows, dtype=torch.int32, device=rt.device)
        with self._workspace(ws):
            self.forward(ctx, cache, greedy)                 # allocates the scratch buffers, loads the kernels
            torch.cuda.synchronize(rt.device)
            before, bounded_before = ops.launches, ops.bounded_launches
            graph = torch.cuda.CUDAGraph()
            collecting = gc.isenabled()
            gc.disable()          # a collection inside the capture could destroy another model's graphs there
            try:
                with torch.cuda.graph(graph):
                    logits = self.forward(ctx, cache, greedy)    # greedy decoding needs no launch after the graph
            finally:
                if collecting:
                    gc.enable()
            kernels = ops.launches - before
        ws.frozen = True
        return _DecodeGraph(rows, graph, stager, ws, logits, greedy, kernels, ops.bounded_launches > bounded_before, kv_limit)

    def _capture_prompt(self, cache: Cache, rows: int) -> _DecodeGraph:
        """Captures a prompt step of `rows` rows (one sequence's piece and its padding sequence). Warm-up and capture
        run in the cache's spare slot and page only."""
        rt = self.rt
        ws = Workspace(rt.device)
        width = sum(cache.groups[gi].max_seq_pages for gi in cache.kv_groups)
        stager = StepStager(rt.device, capacity=3 * rows + 2 * width + 64, fixed=True)
        ctx = stager.stage_prompt_fixed(cache, cache.dummy_slot, [0], 0, rows)
        greedy = torch.empty(1, dtype=torch.int32, device=rt.device)
        with self._workspace(ws):
            self.forward(ctx, cache, greedy)
            torch.cuda.synchronize(rt.device)
            before, bounded_before = ops.launches, ops.bounded_launches
            graph = torch.cuda.CUDAGraph()
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    logits = self.forward(ctx, cache, greedy)
            finally:
                if collecting:
                    gc.enable()
            kernels = ops.launches - before
        ws.frozen = True
        return _DecodeGraph(rows, graph, stager, ws, logits, greedy, kernels, ops.bounded_launches > bounded_before)

    def _prompt_with_graph(self, cache: Cache, slot: int, tokens: Sequence[int], start: int) -> torch.Tensor:
        rows = _prompt_bucket(len(tokens))
        self._graphs_of(cache)                    # (registers the cache's end of life, clears retired graphs)
        per_cache = self._prompt_graphs.setdefault(cache.serial, {})
        g = per_cache.get(rows)
        if g is None:
            g = per_cache[rows] = self._capture_prompt(cache, rows)
            cache._graph_owner = self
        g.stager.stage_prompt_fixed(cache, slot, tokens, start, rows)
        self.last_h2d_bytes = g.stager.last_h2d_bytes
        g.graph.replay()
        ops.launches += g.kernels
        if g.bounded:
            ops.mark_bounded(self.rt.device)
        self.last_greedy = g.greedy          # the row's most likely token, chosen inside the graph
        return g.logits                      # [1, vocab]: the graph's own output buffer, valid until the next step of this size

    def _decode_with_graph(self, cache: Cache, slots, token_lists, want, starts) -> torch.Tensor:
        n = len(slots)
        g = self._decode_graph(cache, _bucket(n), int(np.max(starts)) + 1)
        rows = g.rows
        tokens = [t[0] for t in token_lists]
        batch_key = (tuple(slots), cache.tables_version())
        # the same sequences as in this graph's last step and no page table changed: rewrite tokens and positions only
        if not (g.batch_key == batch_key and g.stager.restage_next_token(tokens, starts)):
            g.stager.stage_decode_fixed(cache, slots, tokens, np.asarray(starts, dtype=np.int64), rows, g.kv_limit)
            g.batch_key = batch_key
        self.last_h2d_bytes = g.stager.last_h2d_bytes
        g.graph.replay()
        ops.launches += g.kernels
        if g.bounded:
            ops.mark_bounded(self.rt.device)
        picked = [i for i, places in enumerate(want) for _ in places]
        if picked == list(range(n)):
            self.last_greedy = g.greedy[:n]
            self._last_graph = g
            return g.logits[:n]          # the graph's own output buffer: valid until the next step of this size
        if not picked:
            return g.logits[:0]
        return g.logits[torch.tensor(picked, dtype=torch.int64, device=self.rt.device)]

    def step_fed(self, cache: Cache, slots: Sequence[int], tokens_dev: torch.Tensor) -> Optional[torch.Tensor]:
        """One more decode step of exactly the sequences of the last step, sequence i fed `tokens_dev[i]` (int32
        on the device: what a sampling kernel chose from the last step's logits), so that the tokens never leave
        the device. Returns the new logits ([n, vocab], the graph's own buffer, with `last_greedy` their argmax),
        or None, with nothing changed, when the last step was no graph step of these sequences with all rows
        wanted, or the cache cannot take another token for every one of them."""
        g = self._last_graph
        n = len(slots)
        if g is None or self.last_greedy is None or g.batch_key is None or g.batch_key[0] != tuple(slots):
            return None
        try:
            starts = cache.begin_step(slots, [1] * n)
        except CacheError:
            return None
        self._uses += 1
        g.last_use = self._uses                  # (so that a capture for another batch does not take this graph for unused)
        if int(np.max(starts)) + 1 > g.kv_limit:
            # the sequences have outgrown the key lengths this graph was sized for: the next graph (tokens_dev, the
            # old graph's buffer, is copied into the new graph's description before `last_greedy` moves on)
            g = self._decode_graph(cache, g.rows, int(np.max(starts)) + 1)
        batch_key = (tuple(slots), cache.tables_version())
        if not (g.batch_key == batch_key and g.stager.restage_fed(tokens_dev, n, starts)):
            g.stager.stage_decode_fixed(cache, slots, [0] * n, np.asarray(starts, dtype=np.int64), g.rows, g.kv_limit)
            g.stager.feed_tokens(tokens_dev, n)
            g.batch_key = batch_key
        self.last_h2d_bytes = g.stager.last_h2d_bytes
        g.graph.replay()
        ops.launches += g.kernels
        if g.bounded:
            ops.mark_bounded(self.rt.device)
        cache.end_step(slots, [1] * n)
        self._last_graph, self.last_greedy = g, g.greedy[:n]
        return g.logits[:n]

    def step_from_last_greedy(self, cache: Cache, slots: Sequence[int]) -> Optional[torch.Tensor]:
        """`step_fed` with the tokens that the last step's graph chose itself (its argmax). Returns the new
        choices (int32 [n] on the device, the graph's own buffer) or None."""
        if self.last_greedy is None or self.step_fed(cache, slots, self.last_greedy) is None:
            return None
        return self.last_greedy

    def forward(self, ctx: StepContext, cache: Cache, greedy: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The step's kernels. `greedy` (int32, one word per wanted row) also takes each returned row's most likely
        token (a soft cap on the logits keeps their order, so it does not matter that it comes after)."""
        rt, spec = self.rt, self.spec
        h = rt.ws.get("stream", (ctx.n_tokens, spec.hidden), torch.float32)
        ops.embed(self.embed, ctx.tokens, h, spec.embed_scale)
        stream = ResidualStream(h, rt)
        last = len(spec.order) - 1
        for i, call in enumerate(spec.order):
            # the norm that reads the stream after this block, for products that carry the norm with them
            next_norm = self.blocks[spec.order[i + 1].layer].first_norm if i < last else self.final_norm
            self.blocks[call.layer].forward(stream, ctx, cache.views[i], next_norm)
        if ctx.want_rows.numel() == 0:
            stream.flush(self.final_norm)
            return torch.empty((0, spec.vocab), dtype=torch.float32, device=rt.device)
        if ctx.want_all and stream.fuses():
            y = stream.norm_input(self.final_norm, lazy=rt.few_rows_shape(ctx.n_tokens, self.head))
        else:
            y = stream.norm(self.final_norm, ctx.want_rows)
        logits = rt.linear(y, self.head, "logits", out_dtype=torch.float32, argmax_into=greedy)
        if spec.logit_cap > 0.0:
            ops.logit_cap(logits, spec.logit_cap)
        return logits


def load_model(folder: str, dtype: str = "bfloat16", device="cuda:0") -> Model:
    """The model a folder's config.json names, with the folder's safetensors."""
    cfg_json = read_json(os.path.join(folder, "config.json"))
    arch = registry.architecture_for(cfg_json)
    config = arch.config_class.from_json(cfg_json)
    spec = config.model_spec()
    weights = load_weights(spec, folder)
    return Model(spec, weights, dtype=dtype, device=device, config=config)
