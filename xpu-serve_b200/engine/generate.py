"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early,
and as many batches one after another as the requests need.

Per sequence the decisions are the reference's (src/engine/engine.cpp:224-362): an empty
prompt or one that does not fit the context is an error; max_new = min(max_new_tokens,
context - prompt); a sampled stop token ends the sequence and is not returned; the token
callback can cancel; reaching max_new ends with "length"; decode time runs from the
first emitted token to the last. What is added is the batch: requests are packed, in
order, into batches that fit the cache; a batch's prompts run in one step (or in pieces
of at most `prefill_chunk` tokens a step), then every live sequence advances by one token
a step; a sequence that ends gives its slot back at once and the others go on.

The loop talks to a `stepper` (engine.engine.DeviceStepper on a GPU; a fake in the tests):
    stepper.max_context, stepper.capacity_tokens, stepper.page_size, stepper.max_slots
    stepper.open(requests) -> handles          one per request, holding a slot
    stepper.close(handles)
    stepper.step(handles, token_lists, want) -> [next token or None per handle]
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional, Sequence

from ..sampling.params import (FINISH_CANCELLED, FINISH_ERROR, FINISH_LENGTH, FINISH_STOP, GenerateRequest,
                               GenerateResult, GenerateStats, TokenCallback)


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def max_new_for(request: GenerateRequest, max_context: int) -> int:
    return max(0, min(request.max_new_tokens, max_context - len(request.prompt)))


def plan_batches(requests: Sequence[GenerateRequest], order: Sequence[int], max_batch: int,
                 capacity_tokens: int, page_size: int, max_context: int) -> List[List[int]]:
    """Packs request indices, in order, into batches whose worst-case token holdings (prompt plus
    max_new, each rounded up to whole pages) fit the cache and whose size is at most max_batch."""
    batches: List[List[int]] = []
    cur: List[int] = []
    held = 0
    for i in order:
        r = requests[i]
        need = _round_up(len(r.prompt) + max_new_for(r, max_context), page_size)
        if cur and (len(cur) >= max_batch or held + need > capacity_tokens):
            batches.append(cur)
            cur, held = [], 0
        cur.append(i)
        held += need
    if cur:
        batches.append(cur)
    return batches


def generate(stepper, requests: Sequence[GenerateRequest], on_token: Optional[TokenCallback] = None,
             max_batch: int = 64, prefill_chunk: int = 8192,
             clock: Callable[[], float] = time.perf_counter) -> List[GenerateResult]:
    results: List[Optional[GenerateResult]] = [None] * len(requests)
    runnable: List[int] = []
    for i, r in enumerate(requests):
        stats = GenerateStats(prompt_tokens=len(r.prompt))
        if len(r.prompt) == 0:
            results[i] = GenerateResult(FINISH_ERROR, [], stats, "empty prompt")
        elif len(r.prompt) >= stepper.max_context:
            results[i] = GenerateResult(FINISH_ERROR, [], stats,
                                        f"prompt of {len(r.prompt)} tokens does not fit the context limit of "
                                        f"{stepper.max_context} tokens")
        elif _round_up(len(r.prompt) + max_new_for(r, stepper.max_context), stepper.page_size) > stepper.capacity_tokens:
            results[i] = GenerateResult(FINISH_ERROR, [], stats,
                                        f"prompt of {len(r.prompt)} tokens plus its output does not fit the cache of "
                                        f"{stepper.capacity_tokens} tokens")
        else:
            try:
                r.sampling.validate()
                runnable.append(i)
            except ValueError as e:
                results[i] = GenerateResult(FINISH_ERROR, [], stats, str(e))
    max_batch = max(1, min(max_batch, stepper.max_slots))
    for batch in plan_batches(requests, runnable, max_batch, stepper.capacity_tokens, stepper.page_size,
                              stepper.max_context):
        _run_batch(stepper, requests, batch, results, on_token, max(1, prefill_chunk), clock)
    return results  # type: ignore[return-value]


def _run_batch(stepper, requests, batch: List[int], results, on_token, prefill_chunk: int, clock) -> None:
    n = len(batch)
    reqs = [requests[i] for i in batch]
    out = [GenerateResult(FINISH_LENGTH, [], GenerateStats(prompt_tokens=len(r.prompt), batch_size=n)) for r in reqs]
    live = list(range(n))          # positions within the batch that still hold a slot
    handles = None
    try:
        handles = stepper.open(reqs)
        max_new = [max_new_for(r, stepper.max_context) for r in reqs]
        # ---- prompts: one step, or pieces of at most prefill_chunk tokens a step
        at = [0] * n
        token: List[Optional[int]] = [None] * n
        t0 = clock()
        while any(at[k] < len(reqs[k].prompt) for k in range(n)):
            left = prefill_chunk
            part, pieces, want = [], [], []
            for k in range(n):
                rest = len(reqs[k].prompt) - at[k]
                if rest <= 0 or left <= 0:
                    continue
                take = min(rest, left)
                left -= take
                part.append(k)
                pieces.append(reqs[k].prompt[at[k]:at[k] + take])
                at[k] += take
                want.append(at[k] == len(reqs[k].prompt) and max_new[k] > 0)
            got = stepper.step([handles[k] for k in part], pieces, want)
            for k, t in zip(part, got):
                if t is not None:
                    token[k] = t
        prefill_ms = (clock() - t0) * 1000.0
        for k in range(n):
            out[k].stats.prefill_ms = prefill_ms
        first_emit = [None] * n
        # ---- decoding: every live sequence by one token a step
        while live:
            ended = []
            for k in list(live):
                r, res = reqs[k], out[k]
                if max_new[k] <= 0:
                    ended.append(k)
                    continue
                t = token[k]
                if t in r.stop_token_ids:
                    res.finish = FINISH_STOP
                    ended.append(k)
                    continue
                now = clock()
                if first_emit[k] is None:
                    first_emit[k] = now
                res.tokens.append(t)
                res.stats.decode_ms = (now - first_emit[k]) * 1000.0
                if on_token is not None and not on_token(batch[k], t):
                    res.finish = FINISH_CANCELLED
                    ended.append(k)
                    continue
                if len(res.tokens) >= max_new[k]:
                    ended.append(k)
            if ended:
                stepper.close([handles[k] for k in ended])
                live = [k for k in live if k not in ended]
            if not live:
                break
            got = stepper.step([handles[k] for k in live], [[token[k]] for k in live], [True] * len(live))
            for k, t in zip(live, got):
                token[k] = t
    except Exception as e:      # the cache may be partly written: every unfinished sequence of the batch fails
        for k in live:
            out[k].finish = FINISH_ERROR
            out[k].error = f"{type(e).__name__}: {e}"
        if handles is not None:
            try:
                stepper.close([handles[k] for k in live])
            except Exception:
                pass
    for k, i in enumerate(batch):
        out[k].stats.generated_tokens = len(out[k].tokens)
        results[i] = out[k]
