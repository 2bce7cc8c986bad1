"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and owns no model code: every step goes through `Model.step` with the
same cache, step function and kernels that generation uses. A trace is a stream of JSON
lines,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` gives each request's next tokens and the places among them whose logits are
wanted; a request seen for the first time gets a free slot; `end` lists requests whose
slots are given back after the step. For a step that wants something, `<out>/<step>.f32`
holds the logits [wanted, vocab] as little-endian float32 in the order of the entries and
of `want`. The nearest thing in the reference is a test helper that collects a prefill's
and then each decoded token's logits (tests/unit/model/step_logits.h:17-47).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO, Optional

import numpy as np

from ..ops import lib as ops
from .model import Model, load_model


class Replayer:
    def __init__(self, model: Model, max_tokens: int, out_dir: Optional[str]):
        self.model = model
        self.cache = model.new_cache(max_tokens)
        self.out_dir = out_dir
        self.slot_of: Dict[str, int] = {}
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)

    def run_step(self, record: dict) -> Optional[np.ndarray]:
        step = record["step"]
        entries = record.get("entries", [])
        ids = [str(e["id"]) for e in entries]
        if len(set(ids)) != len(ids):
            raise ValueError(f"step {step}: a request appears twice")
        new = [i for i in ids if i not in self.slot_of]
        opened = self.cache.open(len(new)) if new else []
        for i, s in zip(new, opened):
            self.slot_of[i] = s
        logits = None
        try:
            if entries:
                slots = [self.slot_of[i] for i in ids]
                tokens = [list(e["tokens"]) for e in entries]
                want = [list(e.get("want", [])) for e in entries]
                out = self.model.step(self.cache, slots, tokens, want)
                if out.shape[0] > 0:
                    logits = out.detach().to("cpu").numpy().astype("<f4", copy=False)
                    dev = self.model.rt.device
                    if ops.tc_status_unread(dev):        # the copy above has waited for the step's kernels
                        ops.tc_status_read(int(ops.gemm_tc_status(dev).item()), dev)
                    if self.out_dir:
                        logits.tofile(os.path.join(self.out_dir, f"{step}.f32"))
        except Exception:
            if opened:       # a refused step leaves no new request behind
                self.cache.close(opened)
                for i in new:
                    del self.slot_of[i]
            raise
        ended = [str(i) for i in record.get("end", [])]
        if ended:
            unknown = [i for i in ended if i not in self.slot_of]
            if unknown:
                raise ValueError(f"step {step}: cannot end unknown request(s) {unknown}")
            self.cache.close([self.slot_of.pop(i) for i in ended])
        return logits


def run(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stream: IO[str] = sys.stdin,
        log: IO[str] = sys.stdout) -> int:
    model = load_model(model_dir, dtype=dtype)
    rp = Replayer(model, max_tokens, out_dir)
    for line in stream:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        rp.run_step(record)
        print(f"done {record['step']}", file=log, flush=True)
    return 0
