#!/usr/bin/env python3
"""Decode and prefill speed of LFM3 at the 1.2B layer shape on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl reference]

A step is one decode step of a batch whose sequences hold 2,048-token prompts (context
4,096). Prints ONE JSON line: decoded tokens a second timed on the device (`value`), the
same through the Python entry point with host tokens in and out (`e2e`), a 2,048-token
prefill (`prefill`), the decode step against the HBM roofline (`roofline`), and decode at
batch 1 and 64 (`points`). Peaks come from MEASURED_PEAKS.json when present. Inputs are
synthetic token ids; every timed step reads all weights (2.3 GB), far more than the 126 MB
L2, so no cache flush is needed between steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The 1.2B family shape: the headline workload
SHAPE_1_2B = {
    "model_type": "lfm3", "vocab_size": 65536, "hidden_size": 2048, "intermediate_size": 8192,
    "num_hidden_layers": 16,
    "layer_types": ["conv", "conv", "attn", "conv", "conv", "attn", "conv", "conv", "attn", "conv", "attn", "conv",
                    "attn", "conv", "attn", "conv"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "conv_L_cache": 3, "conv_bias": False,
    "rope_theta": 1000000.0, "norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_word_embeddings": True,
    "use_sandwich_norm": False, "attn_head_gate": False, "initializer_range": 0.02,
}
PROMPT = 2048
CONTEXT = 4096


def family_shape(layers, hidden, heads, ffn, context, attn_at):
    cfg = dict(SHAPE_1_2B)
    at = set(attn_at)
    cfg.update(num_hidden_layers=layers, layer_types=["attn" if i in at else "conv" for i in range(layers)],
               hidden_size=hidden, num_attention_heads=heads, intermediate_size=ffn, max_position_embeddings=context)
    return cfg


# The 2.6B shape with ragged prompts and the 350M shape at long context: (shape, batch, prompt lengths uniform in [lo, hi], decode steps)
WORKLOADS = {
    "ragged_2.6b": (family_shape(30, 2048, 32, 10752, 8192, range(2, 30, 3)), 16, (256, 4096), 512),
    "long_350m": (family_shape(16, 1024, 16, 6656, 32768, (2, 5, 8, 10, 12, 14)), 64, (1024, 24576), 256),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self._proc = None
        self._paused = False

    def start(self):
        try:
            self._proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                           "--format=csv,noheader,nounits", "-lms", "20"],
                                          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self._proc = None

    def _read(self):
        for line in self._proc.stdout:
            if not self._paused:
                self.rows.append([c.strip() for c in line.split(",")])

    def pause(self):
        self._paused = True

    def resume(self):
        self._paused = False

    def stop(self):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        mhz = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def copy_bandwidth_here() -> float:
    """GB/s of a device-to-device copy of 1 GiB (read + write counted) on this GPU, now: context for the
    roofline fraction when the driver's measured peaks are absent."""
    import torch
    a = torch.empty(1 << 30, dtype=torch.uint8, device="cuda")
    b = torch.empty_like(a)
    for _ in range(2):
        b.copy_(a)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        b.copy_(a)
    e.record()
    torch.cuda.synchronize()
    return 10 * 2 * (1 << 30) / (s.elapsed_time(e) * 1e-3) / 1e9


def model_numbers(cfg: dict, n_layers_run: int):
    """Bytes a decode step must read and flops of a prefill, from the configuration."""
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, D, K = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["conv_L_cache"]
    kinds = cfg["layer_types"][:n_layers_run]
    n_attn = sum(1 for k in kinds if k != "conv")
    n_conv = len(kinds) - n_attn
    ffn = 3 * H * F
    conv = 4 * H * H
    attn = 2 * H * Hq * D + 2 * H * Hkv * D
    layer_params = len(kinds) * ffn + n_conv * conv + n_attn * attn
    weight_bytes = 2 * (layer_params + V * H)              # bfloat16; the tied table is read once, as the head
    kv_bytes_per_token = n_attn * 2 * Hkv * D * 2
    state_bytes = n_conv * (K - 1) * H * 2 * 2              # read and written
    return {"layer_params": layer_params, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "state_bytes": state_bytes, "n_attn": n_attn, "n_conv": n_conv}


def prefill_flops(cfg: dict, nums: dict, T: int) -> float:
    Hq, D, H, V = cfg["num_attention_heads"], cfg["head_dim"], cfg["hidden_size"], cfg["vocab_size"]
    return 2.0 * T * nums["layer_params"] + nums["n_attn"] * 2.0 * T * T * D * Hq + 2.0 * H * V


def synthetic_prompt(V: int, n: int, salt: int):
    return [(salt * 7919 + i * 31 + (i * i) % 11 + 1) % V for i in range(n)]


def time_decode(model, batch: int, steps: int, warmup: int, V: int):
    """Device time of `steps` decode steps (model step + argmax) of `batch` sequences after
    2,048-token prompts. Returns (ms per step, kernel launches per step). More steps than the context
    has room for after the prompt are timed in several runs, each from fresh prompts after its own warm-up."""
    import torch
    from xpu_serve_b200.ops import lib as ops
    room = CONTEXT - PROMPT - warmup - 2
    total_ms, total_launches, left = 0.0, 0, steps
    while left > 0:
        part = min(left, room)
        ms, launches = _time_decode_run(model, batch, part, warmup, V, torch, ops)
        total_ms += ms * part
        total_launches += launches * part
        left -= part
    return total_ms / steps, total_launches / steps


def _time_decode_run(model, batch, steps, warmup, V, torch, ops):
    cache = model.new_cache(batch * CONTEXT, max_slots=batch, max_seq_tokens=CONTEXT)
    slots = cache.open(batch)
    chunk = max(1, 8192 // PROMPT)
    for b0 in range(0, batch, chunk):           # prompts in pieces of at most 8,192 tokens a step
        part = list(range(b0, min(batch, b0 + chunk)))
        model.step(cache, [slots[i] for i in part], [synthetic_prompt(V, PROMPT, i) for i in part],
                   [[] for _ in part])
    out = torch.empty(batch, dtype=torch.int32, device=model.rt.device)
    tokens = [[(7 * i + 3) % V] for i in range(batch)]

    def one():
        logits = model.step(cache, slots, tokens)
        if model.last_greedy is None:         # the decode graph holds the argmax kernel itself
            ops.argmax(logits, out)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    before = ops.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = (ops.launches - before) / steps
    cache.close(slots)
    del cache
    torch.cuda.empty_cache()
    return ms, launches


def time_prefill(model, V: int, warmup: int, runs: int, tokens: int = PROMPT):
    """Median device time (ms) of one prompt of `tokens` tokens in one step."""
    import torch
    cache = model.new_cache(CONTEXT, max_slots=1, max_seq_tokens=CONTEXT)
    times = []
    for r in range(warmup + runs):
        (slot,) = cache.open(1)
        prompt = synthetic_prompt(V, tokens, 100 + r)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        model.step(cache, [slot], [prompt])
        end.record()
        torch.cuda.synchronize()
        if r >= warmup:
            times.append(start.elapsed_time(end))
        cache.close([slot])
    return statistics.median(times)


def time_sampling(rows: int, V: int, runs: int):
    """Device time of the sampling kernel alone on `rows` rows of V random logits, for the usual cuts."""
    import torch
    from xpu_serve_b200.ops import lib as ops
    dev = "cuda:0"
    logits = torch.randn(rows, V, device=dev) * 2.0
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    seeds = torch.arange(rows, dtype=torch.int64, device=dev) + 5
    counters = torch.zeros(rows, dtype=torch.int64, device=dev)
    full = lambda v, dt=torch.float32: torch.full((rows,), v, dtype=dt, device=dev)      # noqa: E731
    cuts = {"temperature": (0.8, 0, 1.0, 0.0), "top_k": (1.0, 50, 1.0, 0.0), "top_p": (0.8, 0, 0.9, 0.0),
            "top_k_top_p_min_p": (0.9, 200, 0.8, 0.01)}
    result = {"only": "sample", "rows": rows, "vocab": V, "unit": "us"}
    for name, (t, k, p, mp) in cuts.items():
        a = (full(t), full(k, torch.int32), full(p), full(mp))
        for _ in range(3):
            ops.sample(logits, *a, seeds, counters, out)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(runs):
            ops.sample(logits, *a, seeds, counters, out)
        end.record()
        torch.cuda.synchronize()
        result[name] = round(start.elapsed_time(end) / runs * 1e3, 1)
    return result


def time_e2e(folder: str, batch: int, steps: int, warmup: int, V: int):
    """The same decode rate through Engine.generate: host token ids in, host token ids out, every
    step with its host-to-device copy of the step's description and its device-to-host copy of the
    chosen tokens."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    engine = Engine(folder, precision="bf16", ctx=CONTEXT, max_tokens=batch * CONTEXT, max_batch=batch)
    reqs = [GenerateRequest(synthetic_prompt(V, PROMPT, 200 + i), SamplingParams(temperature=0.0), steps + warmup + 1, [])
            for i in range(batch)]
    stamps = []

    def on_token(i, t):
        if i == 0:
            stamps.append(time.perf_counter())
        return True

    results = engine.generate(reqs, on_token)
    bad = [r.error for r in results if r.finish == "error"]
    if bad:
        raise RuntimeError(bad[0])
    # request 0's token k arrives after decode step k - 1; skip the warm-up steps
    span = stamps[warmup + steps] - stamps[warmup]
    h2d = engine.model.last_h2d_bytes      # the last decode step's description: tokens, positions, slots, page tables
    return batch * steps / span, h2d, 4 * batch


def measure_workload(name: str, layers=None, batch=None, new=None, repeats: int = 2) -> dict:
    """A batch of unequal prompts through Engine.generate (host token ids in and out): the prompts with one new
    token first (prefill), then the whole workload; decode time is the difference. The last of `repeats` runs."""
    import random
    import torch
    from xpu_serve_b200 import Engine, GenerateRequest, SamplingParams
    from xpu_serve_b200.config import Lfm3Config
    from xpu_serve_b200.weights import write_random_model
    cfg, full_batch, (lo, hi), full_new = WORKLOADS[name]
    cfg = dict(cfg)
    full_layers = cfg["num_hidden_layers"]
    if layers is not None:                       # a smaller case of the same kernels, for profiler captures
        cfg["num_hidden_layers"] = max(1, min(layers, full_layers))
        cfg["layer_types"] = cfg["layer_types"][:cfg["num_hidden_layers"]]
    batch, new = batch or full_batch, new or full_new
    rng = random.Random(3)
    lens = [rng.randint(lo, hi) for _ in range(batch)]
    V = cfg["vocab_size"]
    nums = model_numbers(cfg, cfg["num_hidden_layers"])
    with tempfile.TemporaryDirectory() as root:
        folder = write_random_model(os.path.join(root, name), Lfm3Config.from_json(cfg), seed=0, dtype="bfloat16")
        total = sum(-(-(n + new) // 64) * 64 for n in lens)
        engine = Engine(folder, precision="bf16", ctx=cfg["max_position_embeddings"], max_tokens=total + 64 * batch,
                        max_batch=batch)
    prompts = [synthetic_prompt(V, n, i) for i, n in enumerate(lens)]
    greedy = SamplingParams(temperature=0.0)
    for _ in range(max(1, repeats)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first = engine.generate([GenerateRequest(p, greedy, 1, []) for p in prompts])
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        out = engine.generate([GenerateRequest(p, greedy, new, []) for p in prompts])
        torch.cuda.synchronize()
        t2 = time.perf_counter()
    bad = [r.error for r in first + out if r.finish == "error"]
    if bad:
        raise RuntimeError(bad[0])
    if any(len(r.tokens) != new for r in out) or any(a.tokens[0] != b.tokens[0] for a, b in zip(first, out)):
        raise RuntimeError("the workload's two runs disagree")
    prefill_s = t1 - t0
    decode_s = (t2 - t1) - prefill_s
    step_ms = decode_s / (new - 1) * 1e3
    pk = peaks()
    step_bytes = nums["weight_bytes"] + (sum(lens) + batch * new // 2) * nums["kv_bytes_per_token"] + batch * nums["state_bytes"]
    achieved = step_bytes / (step_ms * 1e-3) / 1e9
    device_gb = round(torch.cuda.max_memory_allocated() / 1e9, 1)
    del engine
    torch.cuda.empty_cache()
    return {
        "workload": name, "metric": "decode tok/s through Engine.generate", "value": round(batch * (new - 1) / decode_s, 1),
        "unit": "tok/s", "ms_per_step": round(step_ms, 4), "decode_steps": new, "dtype": "bf16",
        "data": "synthetic token ids, random weights N(0, 0.02)",
        "prefill": {"value": round(sum(lens) / prefill_s, 1), "tokens": sum(lens), "ms": round(prefill_s * 1e3, 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes), "peaks": pk["source"]},
        "config": {"layers": cfg["num_hidden_layers"], "layers_of_shape": full_layers, "hidden": cfg["hidden_size"],
                   "ffn": cfg["intermediate_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "vocab": V, "attn_layers": nums["n_attn"], "conv_layers": nums["n_conv"], "global_batch": batch,
                   "prompt_min": min(lens), "prompt_max": max(lens), "context": cfg["max_position_embeddings"]},
        "device_gb": device_gb}


def run_workload(name: str, layers=None, batch=None, new=None) -> int:
    print(json.dumps(measure_workload(name, layers, batch, new)))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="default: 256 decode steps, or the workload's own")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=None, help="default: 8, or the workload's own")
    ap.add_argument("--layers", type=int, default=None, help="run only the first N layers (reported in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    ap.add_argument("--skip-family", action="store_true",
                    help="leave out the two other workloads of the family (2.6B shape with unequal prompts, 350M shape "
                         "at long context), which the default run adds to `points`")
    ap.add_argument("--only", default=None, choices=["decode", "prefill", "sample"],
                    help="time one part only and print a short line (for profiler captures)")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="instead of the default run: a batch of unequal prompts at another shape of the family")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "v1k22/xpu-serve is a C++/SYCL program for Intel GPUs with no Python package and no CUDA "
                          "backend; pip cannot install it and its loader refuses this configuration "
                          "(use_sandwich_norm false)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload is not None:
        return run_workload(args.workload, args.layers, args.batch, args.steps)
    args.batch = args.batch or 8
    args.steps = args.steps or 256

    import torch
    from xpu_serve_b200 import load_model
    from xpu_serve_b200.config import Lfm3Config
    from xpu_serve_b200.weights import write_random_model

    if args.only == "sample":
        print(json.dumps(time_sampling(args.batch, SHAPE_1_2B["vocab_size"], args.steps)))
        return 0

    cfg = dict(SHAPE_1_2B)
    full_layers = cfg["num_hidden_layers"]
    n_layers = full_layers if args.layers is None else max(1, min(args.layers, full_layers))
    cfg["num_hidden_layers"] = n_layers
    cfg["layer_types"] = cfg["layer_types"][:n_layers]
    V = cfg["vocab_size"]
    pk = peaks()
    nums = model_numbers(cfg, n_layers)

    with tempfile.TemporaryDirectory() as root:
        folder = write_random_model(os.path.join(root, "lfm3_1_2b"), Lfm3Config.from_json(cfg), seed=0, dtype="bfloat16")
        model = load_model(folder, dtype="bfloat16")

        if args.only == "decode":
            ms, launches = time_decode(model, args.batch, args.steps, args.warmup, V)
            print(json.dumps({"only": "decode", "batch": args.batch, "layers": n_layers, "ms_per_step": round(ms, 4),
                              "launches_per_step": launches, "copy_gbs_here": round(copy_bandwidth_here(), 1)}))
            return 0
        if args.only == "prefill":
            ms = time_prefill(model, V, warmup=args.warmup, runs=args.steps)
            print(json.dumps({"only": "prefill", "layers": n_layers, "tokens": PROMPT, "ms": round(ms, 4)}))
            return 0
        around = ClockSampler()          # clocks during the prefill and the batch 1 / 64 points (`clocks_points`)
        around.start()
        prefill_ms = time_prefill(model, V, warmup=5, runs=9)
        short_ms = time_prefill(model, V, warmup=5, runs=9, tokens=128)
        around.pause()
        pf = prefill_flops(cfg, nums, PROMPT)

        sampler = ClockSampler()
        sampler.start()
        ms, launches = time_decode(model, args.batch, args.steps, args.warmup, V)
        clocks = sampler.stop()

        points = {"prefill_128_ms": round(short_ms, 3)}
        if not args.skip_points:
            around.resume()
            for b in (1, 64):
                pms, _ = time_decode(model, b, max(64, args.steps // 4), 3, V)
                points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
                points[f"decode_b{b}_ms"] = round(pms, 4)
        clocks_points = around.stop()
        del model
        torch.cuda.empty_cache()
        copy_here = copy_bandwidth_here()
        e2e_value, h2d, d2h = time_e2e(folder, args.batch, min(args.steps, CONTEXT - PROMPT - args.warmup - 2), args.warmup, V)
    if not args.skip_family and args.layers is None:
        # the family's two other workloads, through Engine.generate: decode ms a step and fraction of the HBM peak
        for name, key in (("ragged_2.6b", "ragged_2_6b"), ("long_350m", "long_350m")):
            w = measure_workload(name)
            points[f"{key}_tok_s"] = w["value"]
            points[f"{key}_ms"] = w["ms_per_step"]
            points[f"{key}_frac"] = w["roofline"]["frac"]
            points[f"{key}_prefill_tok_s"] = w["prefill"]["value"]

    value = args.batch * 1000.0 / ms
    # the cache grows by one position a step: the timed steps read PROMPT + warmup + steps / 2 positions on average
    kv_positions = PROMPT + args.warmup + min(args.steps, CONTEXT - PROMPT - args.warmup - 2) // 2
    step_bytes = nums["weight_bytes"] + args.batch * (kv_positions * nums["kv_bytes_per_token"] + nums["state_bytes"])
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "LFM3-1.2B-shape decode tok/s (batch 8, 2,048-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {
            "model": "LFM3 1.2B shape", "layers": n_layers, "layers_of_shape": full_layers,
            "hidden": cfg["hidden_size"], "ffn": cfg["intermediate_size"], "vocab": V,
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "conv_kernel": cfg["conv_L_cache"],
            "attn_layers": nums["n_attn"], "conv_layers": nums["n_conv"], "global_batch": args.batch,
            "seq_len": PROMPT, "context": CONTEXT, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (2.3 GB of weights a step)"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "prefill": {"value": round(PROMPT * 1000.0 / prefill_ms, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": step_bytes,
                     "peaks": pk["source"], "copy_gbs_here": round(copy_here, 1)},
        "points": points,
        "clocks": clocks,
        "clocks_points": clocks_points,
        "gpu_launches": int(round(launches * args.steps)),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
