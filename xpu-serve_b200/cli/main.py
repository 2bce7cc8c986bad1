"""Command line in the manner of the reference's `xpu-serve` (src/cli/main.cpp:45-125, 592-671,
896-950): `run`, `bench` and `info` keep its names and option meanings where it has them
(`--precision`, `--ctx`, `--prefill-chunk`, `--max-tokens`, `--temperature`, `--top-k`,
`--top-p`, `--seed`, `--prompt-tokens`, `--gen-tokens`, `--runs`, `--log-level`). There is no
tokenizer here, so `--prompt` takes token ids. `replay` and `random` are this library's own:
trace replay, and writing a model folder with random weights. Unknown options are refused
by name.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    text = text.replace(",", " ")
    try:
        return [int(t) for t in text.split()]
    except ValueError:
        raise SystemExit("--prompt takes token ids separated by spaces or commas (this library has no tokenizer)")


def _engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("model_dir", help="model folder: config.json and *.safetensors")
    p.add_argument("--precision", default="bf16", choices=["bf16", "f32"], help="compute precision")
    p.add_argument("--ctx", type=int, default=8192, help="context length in tokens (prompt + output)")
    p.add_argument("--prefill-chunk", type=int, default=8192, help="tokens per prefill step, over the whole batch")
    p.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache holds (default: ctx x min(batch, 8))")
    p.add_argument("--log-level", default="info", choices=["debug", "info", "warn", "error"])


def _sampling(args, default):
    from ..sampling.params import SamplingParams
    return SamplingParams(
        temperature=default.temperature if args.temperature is None else args.temperature,
        top_k=default.top_k if args.top_k is None else args.top_k,
        top_p=default.top_p if args.top_p is None else args.top_p,
        min_p=default.min_p if args.min_p is None else args.min_p,
        repetition_penalty=default.repetition_penalty if args.repetition_penalty is None else args.repetition_penalty,
        presence_penalty=args.presence_penalty, frequency_penalty=args.frequency_penalty, seed=args.seed)


def cmd_run(args) -> int:
    from ..engine.engine import Engine
    from ..sampling.params import GenerateRequest
    prompts: List[List[int]] = []
    if args.prompt:
        prompts += [_ids(p) for p in args.prompt]
    if args.prompts_file:
        with open(args.prompts_file) as f:
            prompts += [list(map(int, p)) for p in json.load(f)]
    if not prompts:
        raise SystemExit("run needs --prompt (token ids) or --prompts-file (a JSON list of lists of ids)")
    engine = Engine(args.model_dir, precision=args.precision, ctx=args.ctx, max_tokens=args.cache_tokens,
                    max_batch=max(1, min(len(prompts), args.batch)), prefill_chunk=args.prefill_chunk)
    sampling = _sampling(args, engine.default_sampling)
    stops = engine.stop_token_ids if args.stop is None else _ids(args.stop)
    reqs = [GenerateRequest(p, sampling, args.max_tokens, list(stops)) for p in prompts]
    results = engine.generate(reqs)
    for i, r in enumerate(results):
        print(json.dumps({"request": i, "finish": r.finish, "tokens": r.tokens, **({"error": r.error} if r.error else {})}))
        s = r.stats
        if args.log_level in ("debug", "info"):
            print(f"[{s.prompt_tokens} prompt tok, prefill {s.prefill_ms:.1f} ms ({s.prefill_tok_per_s():.1f} tok/s) | "
                  f"{s.generated_tokens} tok, decode {s.decode_tok_per_s():.1f} tok/s, batch {s.batch_size}]",
                  file=sys.stderr)
    return 0 if all(r.finish != "error" for r in results) else 1


def cmd_bench(args) -> int:
    """Prefill and decode speed of synthetic prompts; a different first token per run
    (src/cli/main.cpp:929-936)."""
    from ..engine.engine import Engine
    from ..sampling.params import GenerateRequest, SamplingParams
    engine = Engine(args.model_dir, precision=args.precision, ctx=args.ctx, max_tokens=args.cache_tokens,
                    max_batch=args.batch, prefill_chunk=args.prefill_chunk)
    V = engine.model.spec.vocab
    for run in range(args.runs):
        reqs = []
        for b in range(args.batch):
            prompt = [(run * 7919 + b * 104729 + i * 31 + (i * i) % 11) % V for i in range(args.prompt_tokens)]
            reqs.append(GenerateRequest(prompt, SamplingParams(temperature=0.0), args.gen_tokens, []))
        t0 = time.perf_counter()
        results = engine.generate(reqs)
        wall = time.perf_counter() - t0
        bad = [r.error for r in results if r.finish == "error"]
        if bad:
            raise SystemExit(f"generation failed: {bad[0]}")
        s = results[0].stats
        gen = sum(r.stats.generated_tokens for r in results)
        dec = sum(r.stats.generated_tokens - 1 for r in results) * 1000.0 / s.decode_ms if s.decode_ms > 0 else 0.0
        print(f"run {run}: batch {args.batch}, prompt {s.prompt_tokens} tok, prefill {s.prefill_ms:.1f} ms "
              f"({args.batch * s.prompt_tokens * 1000.0 / s.prefill_ms:.1f} tok/s) | generated {gen} tok, "
              f"decode {dec:.1f} tok/s | wall {wall:.2f} s")
    return 0


def cmd_info(args) -> int:
    from .. import registry
    from ..config.json_util import read_json
    from ..weights.expected import expected_tensors
    cfg_json = read_json(os.path.join(args.model_dir, "config.json"))
    arch = registry.architecture_for(cfg_json)
    spec = arch.config_class.from_json(cfg_json).model_spec()
    tensors = expected_tensors(spec)
    params = sum(int(__import__("math").prod(t.shape)) for t in tensors.values())
    kinds = [l.mixer.kind for l in spec.layers]
    print(json.dumps({"architecture": arch.name, "layers": len(spec.layers), "hidden": spec.hidden,
                      "vocab": spec.vocab, "max_position": spec.max_position, "tied_head": spec.tied_head,
                      "mixers": kinds, "tensors": len(tensors), "parameters": params}, indent=1))
    return 0


def cmd_replay(args) -> int:
    from ..engine.replay import run
    return run(args.model_dir, {"bf16": "bfloat16", "f32": "float32"}[args.precision], args.out, args.max_tokens)


def cmd_random(args) -> int:
    from .. import registry
    from ..config.json_util import read_json
    from ..weights.random_init import write_random_model
    cfg_json = read_json(args.config)
    config = registry.architecture_for(cfg_json).config_class.from_json(cfg_json)
    write_random_model(args.out_dir, config, args.seed, dtype=args.dtype, std=args.std)
    print(args.out_dir)
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="xpu-serve", description="LFM3 on one B200: run | bench | info | replay | random")
    sub = ap.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", aliases=["generate"], help="generate from prompts given as token ids")
    _engine_options(run)
    run.add_argument("--prompt", action="append", help="a prompt as token ids, e.g. \"5 17 3\"; may repeat (one batch)")
    run.add_argument("--prompts-file", help="a JSON list of prompts, each a list of token ids")
    run.add_argument("--max-tokens", type=int, default=1024, help="maximum new tokens per request")
    run.add_argument("--temperature", type=float, default=None, help="sampling temperature (default: the model's)")
    run.add_argument("--top-k", type=int, default=None, help="top-k (default: the model's)")
    run.add_argument("--top-p", type=float, default=None, help="top-p (default: the model's)")
    run.add_argument("--min-p", type=float, default=None, help="min-p (default: the model's)")
    run.add_argument("--repetition-penalty", type=float, default=None)
    run.add_argument("--presence-penalty", type=float, default=0.0)
    run.add_argument("--frequency-penalty", type=float, default=0.0)
    run.add_argument("--seed", type=int, default=None, help="sampling seed")
    run.add_argument("--stop", default=None, help="stop token ids (default: the model's eos ids)")
    run.add_argument("--batch", type=int, default=64, help="most requests in one batch")
    run.set_defaults(fn=cmd_run)

    bench = sub.add_parser("bench", help="prefill and decode speed on synthetic prompts")
    _engine_options(bench)
    bench.add_argument("--prompt-tokens", type=int, default=512, help="prompt length")
    bench.add_argument("--gen-tokens", type=int, default=128, help="tokens to generate")
    bench.add_argument("--runs", type=int, default=3, help="timed runs")
    bench.add_argument("--batch", type=int, default=1, help="requests in the batch")
    bench.set_defaults(fn=cmd_bench)

    info = sub.add_parser("info", help="what a model folder holds")
    info.add_argument("model_dir")
    info.set_defaults(fn=cmd_info)

    replay = sub.add_parser("replay", help="trace replay: JSON steps on standard input, logits to --out")
    replay.add_argument("model_dir")
    replay.add_argument("--precision", default="bf16", choices=["bf16", "f32"])
    replay.add_argument("--out", required=True)
    replay.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (sizes the cache)")
    replay.set_defaults(fn=cmd_replay)

    rnd = sub.add_parser("random", help="write a model folder with random weights")
    rnd.add_argument("out_dir")
    rnd.add_argument("--config", required=True, help="a config.json")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    rnd.add_argument("--std", type=float, default=None, help="standard deviation (default: initializer_range)")
    rnd.set_defaults(fn=cmd_random)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return args.fn(args)
