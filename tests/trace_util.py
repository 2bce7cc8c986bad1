"""Builds replay traces and compares what they give with the plain implementation."""
import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

import plain_lfm3 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole_trace(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole: one step, logits at every place."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_trace(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Each request alone: its head in one step, then its last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def batch_trace(requests: Dict[str, List[int]], batch: int, prompt_frac: float = 0.5) -> List[dict]:
    """Batches of `batch` requests, one batch after another. Each batch starts together: a first step
    with every request's prompt (its first part), then one token each; shorter requests end earlier."""
    steps, n = [], 0
    rids = list(requests)
    for b0 in range(0, len(rids), batch):
        group = rids[b0:b0 + batch]
        heads = {r: max(1, int(len(requests[r]) * prompt_frac)) for r in group}
        entries = [{"id": r, "tokens": requests[r][:heads[r]], "want": list(range(heads[r]))} for r in group]
        ends = [r for r in group if heads[r] == len(requests[r])]
        steps.append({"step": n, "entries": entries, "end": ends})
        n += 1
        at = dict(heads)
        live = [r for r in group if r not in ends]
        while live:
            entries = [{"id": r, "tokens": [requests[r][at[r]]], "want": [0]} for r in live]
            for r in live:
                at[r] += 1
            ends = [r for r in live if at[r] == len(requests[r])]
            steps.append({"step": n, "entries": entries, "end": ends})
            n += 1
            live = [r for r in live if r not in ends]
    return steps


PIECES = (7, 64, 65, 129, 3, 16, 40)


def pieces_trace(requests: Dict[str, List[int]], batch: int, prompt_frac: float = 0.8,
                 pieces: Sequence[int] = PIECES) -> List[dict]:
    """Prompts in pieces, and steps that mix pieces with single tokens. A batch's requests start together with
    the first piece of each; from then on every live request brings, while its prompt (the first
    `prompt_frac` of its tokens) lasts, the next piece of it (sizes cycle through `pieces`, each request
    starting at another place of the cycle), and after that one token a step. So a later piece of a long
    request stands in the same step as single tokens of shorter ones, and shorter requests end earlier."""
    steps, n = [], 0
    rids = list(requests)
    for b0 in range(0, len(rids), batch):
        group = rids[b0:b0 + batch]
        prompt_len = {r: max(1, int(len(requests[r]) * prompt_frac)) for r in group}
        at = {r: 0 for r in group}
        turn = {r: 0 for r in group}
        live = list(group)
        while live:
            entries = []
            for k, r in enumerate(live):
                if at[r] < prompt_len[r]:
                    size = pieces[(turn[r] + (k if turn[r] else 0)) % len(pieces)]
                    take = min(size, prompt_len[r] - at[r])
                    turn[r] += 1
                else:
                    take = 1
                entries.append({"id": r, "tokens": requests[r][at[r]:at[r] + take], "want": list(range(take))})
                at[r] += take
            ends = [r for r in live if at[r] == len(requests[r])]
            steps.append({"step": n, "entries": entries, "end": ends})
            n += 1
            live = [r for r in live if r not in ends]
    return steps


def collect(steps: List[dict], outputs: Dict[int, np.ndarray], vocab: int) -> Dict[Tuple[str, int], np.ndarray]:
    """{(request, position): logits} from the per-step outputs of a trace."""
    pos: Dict[str, int] = {}
    got: Dict[Tuple[str, int], np.ndarray] = {}
    for s in steps:
        rows = outputs.get(s["step"])
        k = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = rows[k]
                k += 1
            pos[e["id"]] = base + len(e["tokens"])
        if rows is not None:
            assert k == rows.shape[0] and rows.shape[1] == vocab
    return got


def run_in_process(replayer, steps: List[dict]) -> Dict[int, np.ndarray]:
    out = {}
    for s in steps:
        r = replayer.run_step(s)
        if r is not None:
            out[s["step"]] = np.array(r, dtype=np.float32)
    return out


def run_program(folder: str, dtype: str, steps: List[dict], out_dir: str, max_tokens: int, vocab: int,
                env=None) -> Dict[int, np.ndarray]:
    """Drives bin/trace_run over its standard input, waiting for `done <step>` after every step."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    out = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not os.path.exists(path)
    return out


def plain_logits(folder: str, requests: Dict[str, List[int]]) -> Dict[Tuple[str, int], np.ndarray]:
    cfg, W = plain.load_folder(folder)
    ref = {}
    for rid, toks in requests.items():
        lg = plain.forward(cfg, W, toks)
        for p in range(len(toks)):
            ref[(rid, p)] = lg[p]
    return ref


def worst_gap(got: Dict, ref: Dict):
    """(largest |difference| / largest |reference logit| over all places, the place, lowest cosine)."""
    scale = max(np.abs(v).max() for v in ref.values())
    worst, where, cos = 0.0, None, 1.0
    assert set(got) == set(ref), f"places differ: {sorted(set(ref) ^ set(got))[:5]}"
    for key in sorted(ref):
        a, b = got[key].astype(np.float64), ref[key]
        assert np.isfinite(a).all(), f"non-finite logits at {key}"
        gap = np.abs(a - b).max() / scale
        if gap > worst:
            worst, where = gap, key
        cos = min(cos, float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300)))
    return worst, where, cos
