"""A plain, slow LFM3 in float64 numpy: whole sequences, no cache, one function per part.

It shares no code with the package: it reads config.json's keys itself and takes tensors
by their checkpoint names. Each function restates a formula of the reference (paths are
relative to the reference project). tests/golden/ holds the logits that the reference's
own CPU backend gives for a tiny random model in its layout; test_plain.py checks this
file against them.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


# ----------------------------------------------------------------------------- reading
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """Every tensor of one safetensors file as float64 (bfloat16 widened exactly)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        raw = data[e["data_offsets"][0]:e["data_offsets"][1]]
        if e["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = u16.view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif e["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2")
        elif e["dtype"] in ("I64", "I32"):
            a = np.frombuffer(raw, dtype="<i8" if e["dtype"] == "I64" else "<i4")
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = a.astype(np.float64).reshape(e["shape"])
    return out


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


def to_bf16(a: np.ndarray) -> np.ndarray:
    """Rounds to bfloat16 (nearest even) and returns float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


# ------------------------------------------------------------------------------- parts
def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """x * (mean(x^2) + eps)^(-1/2) * w over the last axis, no +1 offset
    (src/graph/graph.h:57; src/backend/cpu_ref/ops.cpp:260-281)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def rope_inv_freq(theta: float, head_dim: int, pairs: int) -> np.ndarray:
    """float32 theta^(-2i/head_dim) for i < pairs, 0 beyond (src/models/common/blocks.cpp:131-141)."""
    f = np.zeros(head_dim // 2, dtype=np.float32)
    for i in range(pairs):
        f[i] = np.float32(1.0 / math.pow(theta, (2 * i) / head_dim))
    return f.astype(np.float64)


def rope(x: np.ndarray, pos: np.ndarray, inv_freq: np.ndarray) -> np.ndarray:
    """Rotate-half: pair i couples channels i and i + D/2; angle = pos * inv_freq[i] in float64
    (src/backend/cpu_ref/ops.cpp:375-398). x is [T, heads, D]."""
    half = x.shape[-1] // 2
    ang = pos[:, None].astype(np.float64) * inv_freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s, b * c + a * s], -1)


def causal_conv(g: np.ndarray, w: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
    """conv[t, c] = sum_j w[c, j] * x'[t + j, c] with x' = [K-1 zero rows; g]: w[c, K-1] multiplies
    the current token (src/backend/cpu_ref/ops.cpp:447-471). g is [T, H], w is [H, K]."""
    T, H = g.shape
    K = w.shape[1]
    ext = np.concatenate([np.zeros((K - 1, H)), g], 0)
    out = np.zeros((T, H))
    for j in range(K):
        out += w[:, j][None, :] * ext[j:j + T]
    if bias is not None:
        out = out + bias
    return out


def short_conv(x: np.ndarray, W: Dict[str, np.ndarray], L: str, H: int, K: int, bias: bool) -> np.ndarray:
    """[B | C | X] = in_proj(x); out_proj(C * conv(B * X)) (src/models/lfm3/lfm3_decoder.cpp:94-111)."""
    bcx = x @ W[L + "conv.in_proj.weight"].T
    if bias:
        bcx = bcx + W[L + "conv.in_proj.bias"]
    B, C, X = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    conv = causal_conv(B * X, W[L + "conv.conv.weight"].reshape(H, K), W[L + "conv.conv.bias"] if bias else None)
    out = (C * conv) @ W[L + "conv.out_proj.weight"].T
    if bias:
        out = out + W[L + "conv.out_proj.bias"]
    return out


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int) -> np.ndarray:
    """Causal grouped-query attention of a whole sequence: query t sees key j iff j <= t and
    (window == 0 or t - j < window); head h reads kv head h // (Hq // Hkv); softmax over the
    visible keys (src/backend/cpu_ref/ops.cpp:113-153, 567-592). q [T,Hq,D], k, v [T,Hkv,D]."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    out = np.zeros((T, Hq, D))
    for t in range(T):
        lo = max(0, t - window + 1) if window > 0 else 0
        for h in range(Hq):
            kh = h // (Hq // Hkv)
            s = scale * (k[lo:t + 1, kh] @ q[t, h])
            p = np.exp(s - s.max())
            p /= p.sum()
            out[t, h] = p @ v[lo:t + 1, kh]
    return out


def self_attention(x: np.ndarray, W: Dict[str, np.ndarray], L: str, Hq: int, Hkv: int, D: int, eps: float,
                   inv_freq: np.ndarray, window: int, head_gate: bool, shared_kv=None, return_kv: bool = False):
    """q/k projections -> per-head norms -> RoPE; v raw; attention; sigmoid head gate; o_proj
    (src/models/common/blocks.cpp:143-187; src/models/lfm3/lfm3_decoder.cpp:114-141). With
    `shared_kv` = (k, v) of another call, only q is computed here (blocks.cpp:165-167)."""
    T = x.shape[0]
    pos = np.arange(T)
    A = L + "self_attn."
    q = (x @ W[A + "q_proj.weight"].T).reshape(T, Hq, D)
    q = rope(rms_norm(q, W[A + "q_norm.weight"], eps), pos, inv_freq)
    if shared_kv is not None:
        k, v = shared_kv
    else:
        k = (x @ W[A + "k_proj.weight"].T).reshape(T, Hkv, D)
        v = (x @ W[A + "v_proj.weight"].T).reshape(T, Hkv, D)
        k = rope(rms_norm(k, W[A + "k_norm.weight"], eps), pos, inv_freq)
    o = attention(q, k, v, 1.0 / math.sqrt(D), window)
    if head_gate:
        z = x @ W[A + "gate_proj.weight"].T
        o = o * (1.0 / (1.0 + np.exp(-z)))[:, :, None]
    out = o.reshape(T, Hq * D) @ W[A + "o_proj.weight"].T
    return (out, (k, v)) if return_kv else out


def swiglu(y: np.ndarray, W: Dict[str, np.ndarray], L: str) -> np.ndarray:
    """w2(silu(w1 y) * w3 y), silu(z) = z / (1 + exp(-z)) (src/models/common/blocks.cpp:23-27;
    src/backend/cpu_ref/ops.cpp:242-247)."""
    a = y @ W[L + "feed_forward.w1.weight"].T
    u = y @ W[L + "feed_forward.w3.weight"].T
    return ((a / (1.0 + np.exp(-a))) * u) @ W[L + "feed_forward.w2.weight"].T


# ------------------------------------------------------------------------------- model
def _rope_of(cfg: dict, kind: str, D: int) -> np.ndarray:
    rp = cfg.get("rope_parameters")
    if isinstance(rp, dict) and isinstance(rp.get(kind), dict):
        r = rp[kind]
    elif isinstance(rp, dict) and "rope_theta" in rp:
        r = rp
    else:
        r = {"rope_theta": cfg["rope_theta"]}
    pairs = int(float(r.get("partial_rotary_factor", 1.0)) * D) // 2     # lfm3_config.cpp:20
    return rope_inv_freq(float(r["rope_theta"]), D, pairs)


def forward(cfg: dict, W: Dict[str, np.ndarray], ids: List[int], rows: Optional[Sequence[int]] = None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence from position 0, or of its positions `rows` only
    (layer frame: src/models/lfm3/lfm3_decoder.cpp:49-90; head: src/models/lfm3/lfm3_model.cpp:37-38)."""
    H = cfg["hidden_size"]
    Hq, Hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim", H // Hq)
    K = cfg.get("conv_L_cache", 7)
    eps = cfg["norm_eps"]
    sandwich = cfg.get("use_sandwich_norm", True)
    gate = cfg.get("attn_head_gate", True)
    bias = cfg.get("conv_bias", False)
    tied = cfg.get("tie_embedding", cfg.get("tie_word_embeddings", True))
    P = "model.language_model." if "model.language_model.embed_tokens.weight" in W else "model."
    h = W[P + "embed_tokens.weight"][np.asarray(ids)]
    for i, kind in enumerate(cfg["layer_types"]):
        L = f"{P}layers.{i}."
        x = rms_norm(h, W[L + "operator_norm.weight"], eps)
        if kind == "conv":
            m = short_conv(x, W, L, H, K, bias)
        else:
            sliding = kind == "sliding_attention"
            inv = _rope_of(cfg, "sliding_attention" if sliding else "full_attention", D)
            m = self_attention(x, W, L, Hq, Hkv, D, eps, inv, cfg["sliding_window"] if sliding else 0, gate)
        h = h + (rms_norm(m, W[L + "post_operator_norm.weight"], eps) if sandwich else m)
        y = rms_norm(h, W[L + "ffn_norm.weight"], eps)
        f = swiglu(y, W, L)
        h = h + (rms_norm(f, W[L + "post_ffn_norm.weight"], eps) if sandwich else f)
    if rows is not None:
        h = h[np.asarray(rows, dtype=np.int64)]
    last = rms_norm(h, W[P + "embedding_norm.weight"], eps)
    head = W[P + "embed_tokens.weight"] if tied else W["lm_head.weight"]
    return last @ head.T


# ----------------------------------------------------------------------------- sampling
def _mix64(z: int) -> int:
    m = (1 << 64) - 1
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def uniform(seed: int, counter: int) -> float:
    """The uniform in [0, 1) of (seed, counter): two rounds of the splitmix64 finaliser."""
    m = (1 << 64) - 1
    a = _mix64((seed + 0x9E3779B97F4A7C15) & m)
    b = _mix64(a ^ ((counter * 0xD1342543DE82EF95 + 0x632BE59BD9B4E019) & m))
    return (b >> 11) / 9007199254740992.0


def kept_weights(logits: np.ndarray, temperature: float, top_k: int, top_p: float, min_p: float) -> np.ndarray:
    """Unnormalised probability of each token after the cuts (0 for dropped tokens), following
    src/engine/sampler.cpp:82-132: weight exp((l - max) / T); candidates by descending logit (ties:
    lower id first); top-k keeps k and fixes `total`; the list stops before a weight < min_p and
    after the candidate at which kept / total >= top_p."""
    l = np.asarray(logits, dtype=np.float64)
    V = l.size
    w = np.exp((l - l.max()) / temperature)
    order = np.lexsort((np.arange(V), -l))
    k = min(V, top_k) if top_k > 0 else V
    order = order[:k]
    total = w[order].sum()
    out = np.zeros(V)
    kept = 0.0
    for i, t in enumerate(order):
        if i > 0 and w[t] < min_p:
            break
        out[t] = w[t]
        kept += w[t]
        if top_p < 1.0 and kept / total >= top_p:
            break
    return out


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, min_p: float, u: float) -> int:
    """Greedy when temperature <= 0 or top_k == 1 (first largest, src/engine/sampler.h:36); otherwise
    the token at which the running sum of kept weights, in vocabulary order, passes u * their sum."""
    l = np.asarray(logits, dtype=np.float64)
    if temperature <= 0 or top_k == 1:
        return int(np.argmax(l))
    w = kept_weights(l, temperature, top_k, top_p, min_p)
    target = u * w.sum()
    c = np.cumsum(w)
    idx = int(np.searchsorted(c, target, side="right"))
    nz = np.nonzero(w)[0]
    return int(min(idx, nz[-1]))


def apply_penalties(logits: np.ndarray, prompt: List[int], generated: List[int], repetition: float,
                    presence: float, frequency: float) -> np.ndarray:
    """src/engine/sampler.cpp:20-47."""
    l = np.array(logits, dtype=np.float64)
    if repetition != 1.0:
        for t in set(prompt) | set(generated):
            l[t] = l[t] / repetition if l[t] > 0 else l[t] * repetition
    if presence != 0.0 or frequency != 0.0:
        for t in set(generated):
            l[t] -= presence + frequency * generated.count(t)
    return l
