"""The tiny LFM3 configurations the tests use, and helpers to write them as model folders.

A and B are the two small shapes of the 1.2B family's test plan; they differ in every size and
option (layers, widths that are no power of two, heads and groups, head size, taps, bias,
theta, eps, tied or untied head); C is B without its biases. R is the layout the reference's own loader reads:
sandwich norms, a gate per head, partly rotated heads, a sliding layer whose window is
shorter than the test prompts, 7 taps (tests/parity/model/make_tiny.py:113-140 of the
reference). W adds to B's options a sliding layer with an odd window and two rope bases. X has
widths that are no multiple of 8 and a head size that only the generic attention kernel takes. H has
the head size (64) that the tcgen05 attention kernel takes.
"""
import os

from xpu_serve_b200.config import Lfm3Config
from xpu_serve_b200.weights import write_random_model

CONFIG_A = {
    "model_type": "lfm3", "vocab_size": 512, "hidden_size": 64, "intermediate_size": 192,
    "num_hidden_layers": 4, "layer_types": ["conv", "conv", "attn", "conv"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "conv_L_cache": 3, "conv_bias": False, "rope_theta": 10000.0, "norm_eps": 1e-5,
    "max_position_embeddings": 4096, "tie_word_embeddings": True,
    "use_sandwich_norm": False, "attn_head_gate": False, "initializer_range": 0.02,
}

CONFIG_B = {
    "model_type": "lfm3", "vocab_size": 1000, "hidden_size": 96, "intermediate_size": 320,
    "num_hidden_layers": 6, "layer_types": ["attn", "conv", "conv", "attn", "conv", "attn"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "conv_L_cache": 4, "conv_bias": True, "rope_theta": 500000.0, "norm_eps": 1e-6,
    "max_position_embeddings": 2048, "tie_word_embeddings": False,
    "use_sandwich_norm": False, "attn_head_gate": False, "initializer_range": 0.05,
}

# B without the biases: `conv_bias` is the one option whose formula the reference cannot pin (it refuses the
# key, src/models/lfm3/lfm3_config.cpp:44), so B's other sizes and options are also run without it
CONFIG_C = dict(CONFIG_B, conv_bias=False)

CONFIG_R = {
    "model_type": "lfm3", "vocab_size": 300, "hidden_size": 64, "intermediate_size": 96,
    "num_hidden_layers": 8,
    "layer_types": ["conv", "conv", "full_attention", "conv", "sliding_attention", "conv", "full_attention", "conv"],
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 32,
    "conv_L_cache": 7, "conv_bias": False, "norm_eps": 1e-5, "max_position_embeddings": 1024,
    "sliding_window": 16, "tie_word_embeddings": True, "eos_token_id": 1,
    "rope_parameters": {"full_attention": {"rope_theta": 200.0, "partial_rotary_factor": 0.5},
                        "sliding_attention": {"rope_theta": 50.0}},
}

CONFIG_W = {
    "model_type": "lfm3", "vocab_size": 777, "hidden_size": 80, "intermediate_size": 200,
    "num_hidden_layers": 5,
    "layer_types": ["sliding_attention", "conv", "full_attention", "sliding_attention", "conv"],
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "conv_L_cache": 2, "conv_bias": False, "norm_eps": 3e-6, "max_position_embeddings": 512,
    "sliding_window": 37, "tie_word_embeddings": False, "use_sandwich_norm": True, "attn_head_gate": True,
    "rope_parameters": {"full_attention": {"rope_theta": 1000.0, "partial_rotary_factor": 1.0},
                        "sliding_attention": {"rope_theta": 77.0, "partial_rotary_factor": 0.67}},
}

# widths that are no multiple of 8 (none of the 16-byte vector paths applies), a vocabulary that is odd
CONFIG_X = {
    "model_type": "lfm3", "vocab_size": 1001, "hidden_size": 100, "intermediate_size": 250,
    "num_hidden_layers": 3, "layer_types": ["conv", "full_attention", "conv"],
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 80,
    "conv_L_cache": 5, "conv_bias": True, "norm_eps": 1e-5, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "use_sandwich_norm": False, "attn_head_gate": True,
    "rope_parameters": {"full_attention": {"rope_theta": 5000.0, "partial_rotary_factor": 0.25}},
}

# head size 64 with two heads a group: in bfloat16 its prompts take the tcgen05 attention kernel (full and
# sliding layers, a gate per head), its single tokens the mma.sync decode kernel
CONFIG_H = {
    "model_type": "lfm3", "vocab_size": 400, "hidden_size": 128, "intermediate_size": 256,
    "num_hidden_layers": 3, "layer_types": ["full_attention", "conv", "sliding_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "conv_L_cache": 3, "conv_bias": False, "norm_eps": 1e-5, "max_position_embeddings": 1024,
    "sliding_window": 50, "tie_word_embeddings": True, "use_sandwich_norm": False, "attn_head_gate": True,
    "rope_parameters": {"full_attention": {"rope_theta": 10000.0, "partial_rotary_factor": 1.0},
                        "sliding_attention": {"rope_theta": 300.0, "partial_rotary_factor": 0.5}},
}

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "R": CONFIG_R, "W": CONFIG_W, "X": CONFIG_X, "H": CONFIG_H}
SEEDS = {"A": 0, "B": 1, "C": 1, "R": 2, "W": 3, "X": 4, "H": 5}
# Plain N(0, sigma) weights give near-uniform attention and near-linear layers. These factors make the
# parts matter: q and k large enough for peaked scores, taps and gates of order one.
LIVELY = {"q_proj.weight": 6.0, "k_proj.weight": 6.0, "conv.conv.weight": 12.0, "gate_proj.weight": 8.0,
          "embed_tokens.weight": 10.0}


def make_folder(root, name: str, dtype: str = "float32", lively: bool = True) -> str:
    """Writes configuration `name` with random weights under `root` and returns the folder."""
    cfg = Lfm3Config.from_json(CONFIGS[name])
    folder = os.path.join(str(root), f"lfm3_{name}_{dtype}")
    if not os.path.isfile(os.path.join(folder, "model.safetensors")):
        write_random_model(folder, cfg, SEEDS[name], dtype=dtype,
                           norm_range=(0.5, 1.5) if lively else None,
                           scale=LIVELY if lively else None)
    return folder


def prompt(name: str, length: int, salt: int = 0):
    V = CONFIGS[name]["vocab_size"]
    return [(i * 37 + 5 + 11 * salt + (i * i) % 7) % V for i in range(length)]


# ---------------------------------------------------------------------------------------------- bounds
# Largest |difference| over largest |reference logit|, engine against the plain float64 implementation.
# Upper limits. float32: 1e-5, the target of the 32-bit path. bfloat16: a value is rounded to 8 significant bits
# (relative error up to u = 2^-9) about ten times a layer (normed input, projections, mixer state and output,
# gate/up, activation, branch output); independent roundings add like a random walk, so a logit's typical error
# is about sqrt(10 * layers) * u of the logits' scale, and the largest of some 10^5 logits lies a few times
# higher: 4 * sqrt(10 * layers) * u.
# Measured on a B200, the worst of the replay schedules (whole, last 32 one by one, batches of 3 / 5 / 11,
# prompts in pieces) per configuration; a test's bound is three times that, capped by the upper limit, so that
# a fault that costs a configuration a few times its usual error fails the test.
U_BF16 = 2.0 ** -9
MEASURED_GAP = {
    "float32": {"A": 2.0e-7, "B": 3.2e-7, "C": 2.9e-7, "R": 1.9e-6, "W": 1.2e-6, "X": 2.2e-7, "H": 1.9e-7},
    "bfloat16": {"A": 1.1e-3, "B": 4.4e-3, "C": 4.1e-3, "R": 2.9e-2, "W": 1.9e-2, "X": 8.7e-4, "H": 7.5e-4},
}


def upper_limit(layers: int, dtype: str) -> float:
    return 1e-5 if dtype == "float32" else 4.0 * (10.0 * layers) ** 0.5 * U_BF16


def bound(name: str, dtype: str) -> float:
    return min(upper_limit(CONFIGS[name]["num_hidden_layers"], dtype), 3.0 * MEASURED_GAP[dtype][name])
