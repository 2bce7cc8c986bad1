"""`bin/xpu-serve run` and `bench` as programs (src/cli/main.cpp:592-671, 896-950), with a model folder's
generation defaults: greedy because generation_config.json does not ask for sampling, stopped by its
`eos_token_id`, by config.json's, or by `--stop` in their place."""
import json
import os
import re
import subprocess
import sys

import pytest

import plain_lfm3 as plain
import tiny
from test_generate_gpu import plain_greedy

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = [sys.executable, os.path.join(ROOT, "bin", "xpu-serve")]


def run_cli(*args, env=None):
    p = subprocess.run(CLI + [str(a) for a in args], capture_output=True, text=True, timeout=300,
                       env=None if env is None else dict(os.environ, **env))
    return p.returncode, p.stdout, p.stderr


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    """Configuration B in float32, its free greedy run from one prompt, and a place k in that run whose token
    has not come before (so that it can serve as a stop token)."""
    from xpu_serve_b200.config import Lfm3Config
    from xpu_serve_b200.weights import write_random_model
    root = tmp_path_factory.mktemp("cli")
    base = tiny.make_folder(root, "B", "float32")
    cfg, W = plain.load_folder(base)
    prompt = tiny.prompt("B", 11, salt=91)
    free, margins = plain_greedy(cfg, W, prompt, 16)
    assert min(margins) > 1e-3, "the test's own tokens are near ties; pick another prompt"
    k = next(i for i in range(4, 16) if free[i] not in free[:i])
    j = next(i for i in range(1, k) if free[i] not in free[:i])
    folder = write_random_model(str(root / "with_defaults"), Lfm3Config.from_json(dict(tiny.CONFIG_B, eos_token_id=free[k])),
                                tiny.SEEDS["B"], dtype="float32", norm_range=(0.5, 1.5), scale=tiny.LIVELY,
                                generation={"temperature": 0.7, "top_k": 5})          # no do_sample: greedy
    sampled = write_random_model(str(root / "sampled"), Lfm3Config.from_json(tiny.CONFIG_B), tiny.SEEDS["B"],
                                 dtype="float32", norm_range=(0.5, 1.5), scale=tiny.LIVELY,
                                 generation={"do_sample": True, "temperature": 0.8, "top_k": 1, "eos_token_id": [free[j]]})
    return {"folder": folder, "sampled": sampled, "prompt": prompt, "free": free, "k": k, "j": j}


def test_run_stops_at_the_folder_s_eos(model):
    rc, out, err = run_cli("run", model["folder"], "--prompt", " ".join(map(str, model["prompt"])), "--max-tokens", 16,
                           "--precision", "f32", "--ctx", 128)
    assert rc == 0, err
    res = json.loads(out.strip().splitlines()[-1])
    assert res["finish"] == "stop" and res["tokens"] == model["free"][:model["k"]]
    assert re.search(r"\[11 prompt tok, prefill [\d.]+ ms .* tok, decode [\d.]+ tok/s, batch 1\]", err)


def test_stop_option_takes_the_place_of_the_folder_s_ids(model):
    free, j = model["free"], model["j"]
    rc, out, err = run_cli("run", model["folder"], "--prompt", ",".join(map(str, model["prompt"])), "--max-tokens", 16,
                           "--precision", "f32", "--ctx", 128, "--stop", str(free[j]), "--log-level", "error")
    assert rc == 0, err
    res = json.loads(out.strip().splitlines()[-1])
    assert res["finish"] == "stop" and res["tokens"] == free[:j]
    assert "prompt tok" not in err
    # a stop id that never comes: the run goes past the folder's own eos to its length
    rc, out, err = run_cli("run", model["folder"], "--prompt", " ".join(map(str, model["prompt"])), "--max-tokens", 16,
                           "--precision", "f32", "--ctx", 128, "--stop", str(tiny.CONFIG_B["vocab_size"] - 1))
    res = json.loads(out.strip().splitlines()[-1])
    assert rc == 0 and res["finish"] == "length" and res["tokens"] == free


def test_generation_config_s_eos_and_sampling_defaults(model):
    """do_sample with top_k 1 is greedy again (src/engine/sampler.h:36); the file's eos list ends the run; two
    prompts make one batch; --temperature 0 on the command line overrides the file."""
    free, j = model["free"], model["j"]
    other = tiny.prompt("B", 6, salt=92)
    rc, out, err = run_cli("run", model["sampled"], "--prompt", " ".join(map(str, model["prompt"])), "--prompt",
                           " ".join(map(str, other)), "--max-tokens", 16, "--precision", "f32", "--ctx", 128,
                           "--temperature", 0)
    assert rc == 0, err
    lines = [json.loads(l) for l in out.strip().splitlines()]
    assert [l["request"] for l in lines] == [0, 1]
    assert lines[0]["finish"] == "stop" and lines[0]["tokens"] == free[:j]
    assert "batch 2" in err


def test_run_refuses_what_it_cannot_do(model):
    rc, out, err = run_cli("run", model["folder"], "--max-tokens", 4)
    assert rc != 0 and "--prompt" in err
    rc, out, err = run_cli("run", model["folder"], "--prompt", "hello world")
    assert rc != 0 and "token ids" in err
    rc, out, err = run_cli("run", model["folder"], "--prompt", "1 2 99999", "--precision", "f32", "--ctx", 64)
    res = json.loads(out.strip().splitlines()[-1])
    assert rc == 1 and res["finish"] == "error" and "99999" in res["error"]


def test_bench_prints_a_line_a_run(model):
    rc, out, err = run_cli("bench", model["folder"], "--prompt-tokens", 24, "--gen-tokens", 8, "--runs", 3, "--ctx", 128)
    assert rc == 0, err
    lines = [l for l in out.strip().splitlines() if l.startswith("run ")]
    assert len(lines) == 3
    for i, l in enumerate(lines):
        m = re.match(rf"run {i}: batch 1, prompt 24 tok, prefill [\d.]+ ms \([\d.]+ tok/s\) \| generated 8 tok, "
                     r"decode ([\d.]+) tok/s \| wall [\d.]+ s", l)
        assert m and float(m.group(1)) > 0, l


def test_profile_and_sync_switches(model):
    """XS_PROFILE=1 times every launch with CUDA events and prints the sums by kernel and sizes at exit; XS_SYNC=1
    waits for the device after every launch (an error would carry the launch's name). Neither changes a token."""
    args = ("run", model["folder"], "--prompt", " ".join(map(str, model["prompt"])), "--max-tokens", 16, "--precision", "bf16",
            "--ctx", 128, "--log-level", "error")
    rc, out, err = run_cli(*args)
    assert rc == 0, err
    plain_run = json.loads(out.strip().splitlines()[-1])
    rc, out, err = run_cli(*args, env={"XS_PROFILE": "1"})
    assert rc == 0, err
    assert json.loads(out.strip().splitlines()[-1]) == plain_run
    head = re.search(r"\[xpu_serve_b200 profile\] (\d+) launches, (\d+) us on the device", err)
    assert head and int(head.group(1)) > 50 and int(head.group(2)) > 0, err[-2000:]
    rows = re.findall(r"^\s+([\d.]+) us\s+([\d.]+) %\s+x(\d+)\s+(xs_\w+) \(([\d, -]*)\)", err, flags=re.M)
    names = {r[3] for r in rows}
    assert {"xs_gemm_small_m_ex", "xs_embed", "xs_qk_norm_rope_store"} <= names, names
    assert abs(sum(float(r[1]) for r in rows) - 100.0) < 1.0
    rc, out, err = run_cli(*args, env={"XS_SYNC": "1"})
    assert rc == 0, err
    assert json.loads(out.strip().splitlines()[-1]) == plain_run
