"""The command line's parser and the commands that need no GPU (`random`, `info`), and a model folder's
generation defaults and stop ids (src/cli/main.cpp:72-125, src/cli/args.cpp:44,
src/models/config_util.cpp:162-182, src/models/lfm3/lfm3_model.cpp:69-77)."""
import json
import os

import pytest

import tiny
from xpu_serve_b200.cli.main import build_parser, main
from xpu_serve_b200.config import Lfm3Config
from xpu_serve_b200.sampling.params import SamplingParams, merged_stop_ids, read_generation_defaults


def test_unknown_options_are_refused_by_name(capsys):
    for argv in (["run", "folder", "--bogus", "1"], ["bench", "folder", "--prompt-tokens", "8", "--nope"],
                 ["info", "folder", "--verbose"], ["replay", "folder", "--out", "o", "--max-tokens", "64", "--fast"]):
        with pytest.raises(SystemExit) as e:
            build_parser().parse_args(argv)
        assert e.value.code == 2
        err = capsys.readouterr().err
        bad = [a for a in argv if a.startswith("--")][-1]
        assert bad in err, f"the refusal does not name {bad}: {err}"


def test_the_reference_s_option_names_and_defaults():
    run = build_parser().parse_args(["run", "m", "--prompt", "1 2 3"])
    assert (run.max_tokens, run.ctx, run.precision, run.prefill_chunk) == (1024, 8192, "bf16", 8192)
    assert run.temperature is None and run.top_k is None and run.top_p is None and run.seed is None
    bench = build_parser().parse_args(["bench", "m"])
    assert (bench.prompt_tokens, bench.gen_tokens, bench.runs) == (512, 128, 3)
    gen = build_parser().parse_args(["generate", "m", "--prompt", "5,17,3", "--temperature", "0.7", "--top-k", "40",
                                     "--top-p", "0.9", "--seed", "3", "--precision", "f32", "--ctx", "256"])
    assert (gen.temperature, gen.top_k, gen.top_p, gen.seed, gen.precision, gen.ctx) == (0.7, 40, 0.9, 3, "f32", 256)
    with pytest.raises(SystemExit):
        build_parser().parse_args(["run", "m", "--precision", "f16"])


def test_random_then_info(tmp_path, capsys):
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny.CONFIG_R))
    out = str(tmp_path / "model")
    assert main(["random", out, "--config", str(cfg_path), "--seed", "5", "--dtype", "float32"]) == 0
    assert capsys.readouterr().out.strip() == out
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    assert main(["info", out]) == 0
    info = json.loads(capsys.readouterr().out)
    cfg = Lfm3Config.from_json(tiny.CONFIG_R)
    H, F, V, K = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.conv_L_cache
    qd, kd = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    conv = 3 * H * H + H * K + H * H
    attn = qd * H + 2 * kd * H + H * qd + cfg.num_attention_heads * H + 2 * cfg.head_dim
    per_layer = 3 * H * F + 4 * H
    n_conv = sum(1 for k in cfg.layer_types if k == "conv")
    want = V * H + H + len(cfg.layer_types) * per_layer + n_conv * conv + (len(cfg.layer_types) - n_conv) * attn
    assert info["architecture"] == "lfm3" and info["layers"] == 8 and info["vocab"] == V and info["tied_head"]
    assert info["mixers"] == ["short_conv", "short_conv", "attention", "short_conv", "attention", "short_conv",
                              "attention", "short_conv"]
    assert info["parameters"] == want
    # the folder reads back to the configuration it was written from, eos id included
    assert Lfm3Config.from_json(json.loads(open(os.path.join(out, "config.json")).read())) == cfg


def write_gen(folder, obj):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "generation_config.json"), "w") as f:
        json.dump(obj, f)
    return str(folder)


def test_generation_defaults(tmp_path):
    # no file: the defaults stand, no stop ids
    p, stops = read_generation_defaults(str(tmp_path))
    assert p == SamplingParams() and stops == []
    # do_sample absent or false: greedy, whatever temperature says; the cuts are still read
    p, stops = read_generation_defaults(write_gen(tmp_path / "a", {"temperature": 0.6, "top_k": 50, "eos_token_id": 7}))
    assert p.temperature == 0.0 and p.greedy() and p.top_k == 50 and stops == [7]
    p, _ = read_generation_defaults(write_gen(tmp_path / "b", {"do_sample": False, "temperature": 0.9}))
    assert p.temperature == 0.0
    # do_sample true: the file's values, the defaults where it has none
    p, stops = read_generation_defaults(write_gen(tmp_path / "c", {
        "do_sample": True, "temperature": 0.3, "top_k": 20, "top_p": 0.85, "min_p": 0.05, "repetition_penalty": 1.1,
        "eos_token_id": [9, 2, 9]}))
    assert (p.temperature, p.top_k, p.top_p, p.min_p, p.repetition_penalty) == (0.3, 20, 0.85, 0.05, 1.1)
    assert stops == [9, 2, 9] and p.presence_penalty == 0.0 and p.seed is None
    p, _ = read_generation_defaults(write_gen(tmp_path / "d", {"do_sample": True}))
    assert p.temperature == 1.0 and p.top_k == 0 and p.top_p == 1.0
    # values of the wrong type are passed over as the reference passes them over (is_number checks)
    p, _ = read_generation_defaults(write_gen(tmp_path / "e", {"do_sample": True, "temperature": "hot", "top_k": 2.5, "top_p": True}))
    assert p.temperature == 1.0 and p.top_k == 0 and p.top_p == 1.0


def test_stop_ids_are_merged_from_both_files(tmp_path):
    cfg = Lfm3Config.from_json(dict(tiny.CONFIG_R, eos_token_id=[4, 1]))
    assert cfg.eos_token_id == (4, 1)
    assert merged_stop_ids(str(tmp_path), cfg) == [1, 4]                       # config.json alone
    folder = write_gen(tmp_path / "g", {"eos_token_id": [7, 4]})
    assert merged_stop_ids(folder, cfg) == [1, 4, 7]                           # both, sorted, each once
    assert merged_stop_ids(folder, Lfm3Config.from_json(tiny.CONFIG_A)) == [4, 7]
    assert merged_stop_ids(str(tmp_path), Lfm3Config.from_json(tiny.CONFIG_A)) == []
    assert Lfm3Config.from_json(dict(tiny.CONFIG_A, eos_token_id=3)).eos_token_id == (3,)   # a number or a list
