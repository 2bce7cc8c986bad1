"""Safetensors by name, the one error that lists everything wrong, random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_lfm3 as plain
import tiny
from xpu_serve_b200.config import Lfm3Config
from xpu_serve_b200.weights import (WeightError, WeightStore, expected_tensors, load_weights, random_tensors,
                                    write_random_model, write_safetensors)


def test_write_read_round_trip(tmp_path):
    a = torch.randn(3, 5)
    b = torch.randn(7).to(torch.bfloat16)
    c = torch.arange(6, dtype=torch.int64).reshape(2, 3)
    write_safetensors(str(tmp_path / "model.safetensors"), [("a", a), ("b", b), ("c", c)])
    store = WeightStore.open_dir(str(tmp_path))
    assert set(store.names()) == {"a", "b", "c"}
    assert torch.equal(store.get("a"), a) and torch.equal(store.get("b"), b) and torch.equal(store.get("c"), c)
    assert store.dtype("b") == torch.bfloat16 and store.shape("c") == (2, 3)
    other = plain.read_safetensors(str(tmp_path / "model.safetensors"))
    assert np.array_equal(other["b"], b.to(torch.float64).numpy())


def test_header_errors_name_the_file(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"1234")
    with pytest.raises(WeightError, match="not a safetensors file"):
        WeightStore.open_dir(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(WeightError, match="header length 1000"):
        WeightStore.open_dir(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(WeightError, match="invalid safetensors header"):
        WeightStore.open_dir(str(tmp_path))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(WeightError, match="'t' is 12 bytes but .* needs 16"):
        WeightStore.open_dir(str(tmp_path))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightError, match="invalid data_offsets"):
        WeightStore.open_dir(str(tmp_path))
    os.remove(p)
    with pytest.raises(WeightError, match="no safetensors files"):
        WeightStore.open_dir(str(tmp_path))


def test_duplicate_name_across_files(tmp_path):
    write_safetensors(str(tmp_path / "a.safetensors"), [("x", torch.zeros(2))])
    write_safetensors(str(tmp_path / "b.safetensors"), [("x", torch.zeros(2))])
    with pytest.raises(WeightError, match="'x' appears in more than one"):
        WeightStore.open_dir(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Lfm3Config.from_json(tiny.CONFIG_A)
    spec = cfg.model_spec()
    tensors = dict(random_tensors(spec, 0, "float32"))
    del tensors["model.layers.2.self_attn.k_norm.weight"]
    del tensors["model.layers.0.conv.in_proj.weight"]
    tensors["model.layers.1.conv.conv.weight"] = torch.zeros(64, 3)          # [H, K] instead of [H, 1, K]
    tensors["model.layers.3.feed_forward.w2.weight"] = torch.zeros(192, 64)  # transposed
    tensors["model.layers.2.self_attn.gate_proj.weight"] = torch.zeros(4, 64)  # this configuration has no gate
    tensors["lm_head.weight"] = torch.zeros(512, 64)                          # tied: no head expected
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as e:
        load_weights(spec, str(tmp_path))
    msg = str(e.value)
    assert "missing (2)" in msg and "k_norm.weight" in msg and "conv.in_proj.weight" in msg
    assert "unexpected (2)" in msg and "gate_proj.weight" in msg and "lm_head.weight" in msg
    assert "wrong shape (2)" in msg and "[64, 3], expected [64, 1, 3]" in msg and "[192, 64], expected [64, 192]" in msg


def test_stored_types_are_kept(tmp_path):
    cfg = Lfm3Config.from_json(tiny.CONFIG_B)
    folder = write_random_model(str(tmp_path / "b"), cfg, 1, dtype="bfloat16")
    w = load_weights(cfg.model_spec(), folder)
    assert w["embed_tokens.weight"].dtype == torch.bfloat16           # 16-bit stays 16-bit
    assert w["layers.0.operator_norm.weight"].dtype == torch.float32  # stored in 32 bits, stays so
    assert w["lm_head.weight"].shape == (1000, 96)
    assert "model.embed_tokens.weight" not in w


def test_random_mode_is_seeded_and_counter_based(tmp_path):
    spec = Lfm3Config.from_json(tiny.CONFIG_A).model_spec()
    a = dict(random_tensors(spec, 5, "float32"))
    b = dict(random_tensors(spec, 5, "float32"))
    c = dict(random_tensors(spec, 6, "float32"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert list(a) == list(expected_tensors(spec))
    e = a["model.embed_tokens.weight"]
    assert abs(float(e.std()) - 0.02) < 0.001 and torch.equal(a["model.embedding_norm.weight"], torch.ones(64))
    wide = Lfm3Config.from_json(dict(tiny.CONFIG_A, intermediate_size=256)).model_spec()
    d = dict(random_tensors(wide, 5, "float32"))
    assert torch.equal(a["model.embed_tokens.weight"], d["model.embed_tokens.weight"])      # same index, same draw
    assert torch.equal(a["model.layers.0.conv.in_proj.weight"], d["model.layers.0.conv.in_proj.weight"])


def test_folder_holds_config_and_weights(tmp_path):
    cfg = Lfm3Config.from_json(tiny.CONFIG_W)
    folder = write_random_model(str(tmp_path / "w"), cfg, 3, dtype="float32")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    with open(os.path.join(folder, "config.json")) as f:
        assert Lfm3Config.from_json(json.load(f)) == cfg
    load_weights(cfg.model_spec(), folder)


def test_vl_prefix_is_probed(tmp_path):
    cfg = Lfm3Config.from_json(tiny.CONFIG_A)
    spec = cfg.model_spec()
    renamed = [(n.replace("model.", "model.language_model.", 1), t) for n, t in random_tensors(spec, 0, "float32")]
    write_safetensors(str(tmp_path / "model.safetensors"), renamed)
    w = load_weights(spec, str(tmp_path))
    assert "embed_tokens.weight" in w and "layers.3.conv.out_proj.weight" in w


def test_a_wrapped_checkpoint_may_hold_other_towers(tmp_path):
    """An lfm3_vl checkpoint keeps the text decoder under model.language_model. beside vision tensors
    (src/models/lfm3/lfm3_decoder.cpp:14-19). Those are not this model's: it loads. A stray tensor under the
    decoder's own prefix is still named, and so is any stray tensor of a plain checkpoint."""
    import torch
    cfg = Lfm3Config.from_json(tiny.CONFIG_A)
    spec = cfg.model_spec()
    renamed = [(n.replace("model.", "model.language_model.", 1), t) for n, t in random_tensors(spec, 0, "float32")]
    extra = [("model.vision_tower.patch_embed.weight", torch.zeros(4, 4)), ("model.multi_modal_projector.w", torch.zeros(2))]
    for d in ("vl", "vl2", "plain"):
        os.makedirs(tmp_path / d)
    write_safetensors(str(tmp_path / "vl" / "model.safetensors"), renamed + extra)
    w = load_weights(spec, str(tmp_path / "vl"))
    assert "embed_tokens.weight" in w and not any("vision" in k for k in w)
    write_safetensors(str(tmp_path / "vl2" / "model.safetensors"),
                      renamed + extra + [("model.language_model.layers.0.stray.weight", torch.zeros(3))])
    with pytest.raises(WeightError, match=r"unexpected \(1\): model.language_model.layers.0.stray.weight"):
        load_weights(spec, str(tmp_path / "vl2"))
    write_safetensors(str(tmp_path / "plain" / "model.safetensors"), list(random_tensors(spec, 0, "float32")) + extra[:1])
    with pytest.raises(WeightError, match=r"unexpected \(1\): model.vision_tower.patch_embed.weight"):
        load_weights(spec, str(tmp_path / "plain"))
