"""Grouped-query attention over the paged cache, with per-head q/k norms, rotary position
encoding and an optional sigmoid gate per head (src/models/common/blocks.cpp:143-187,
src/models/lfm3/lfm3_decoder.cpp:114-141).

One matrix product gives q, k, v and the gate logits: the four weights are stacked at
load ([q; k; v; gate], the gate rows padded to a multiple of 8). The cache keeps normed,
rotated keys and raw values. A call that reads another call's cache computes q (and the
gate) only.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import KVNeed, Mixer, TensorSpec


def decode_splits(tiles: int, blocks: int, slots: int, fixed: float = 2.0) -> int:
    """Into how many parts to cut each sequence's keys when every sequence brings one token: `tiles` CTAs
    (sequences x kv heads) would each walk `blocks` 64-key blocks; `slots` CTAs run at one time. The cost of a
    choice is its number of rounds of CTAs times a CTA's length (its blocks and a fixed cost worth about two),
    plus the combine kernel when there is more than one part, which walks the parts one after another (a third
    of a block each; measured on B200: one sequence of 2,048 keys takes 9 us in 8 parts, 13 us in 32).
    64 sequences of 2,048 keys over 444 slots: one part is 2 rounds of 35, four parts are 5 rounds of 11."""
    best, best_cost = 1, None
    for parts in range(1, max(1, min(blocks, 64)) + 1):
        rounds = -(-tiles * parts // slots)
        cost = rounds * (-(-blocks // parts) + fixed) + (1.5 + parts / 3.0 if parts > 1 else 0.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = parts, cost
    return best


class AttentionMixer(Mixer):
    kind = "attention"
    fuses_norm = True
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        qd, kd = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        out = {
            n["q"]: TensorSpec((qd, spec.hidden)), n["k"]: TensorSpec((kd, spec.hidden)),
            n["v"]: TensorSpec((kd, spec.hidden)), n["o"]: TensorSpec((spec.hidden, qd)),
        }
        if spec.head_gate:
            out[n["gate"]] = TensorSpec((spec.heads, spec.hidden))
        if spec.qk_norm:
            out[n["q_norm"]] = TensorSpec((spec.head_dim,), init="ones", role="vector")
            out[n["k_norm"]] = TensorSpec((spec.head_dim,), init="ones", role="vector")
        if spec.qkv_bias:
            out[n["q_bias"]] = TensorSpec((qd,), init="zeros", role="vector")
            out[n["k_bias"]] = TensorSpec((kd,), init="zeros", role="vector")
            out[n["v_bias"]] = TensorSpec((kd,), init="zeros", role="vector")
        return out

    @classmethod
    def cache_need(cls, spec):
        return KVNeed(spec.kv_heads, spec.head_dim, spec.window)

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.head_dim % 2 != 0 or spec.head_dim > 256:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be even and at most 256")
        if spec.heads % spec.kv_heads != 0:
            raise ValueError(f"attention: {spec.heads} heads over {spec.kv_heads} kv heads")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.q_dim = spec.heads * spec.head_dim
        self.kv_dim = spec.kv_heads * spec.head_dim
        # A checkpoint whose rotation couples channels 2i and 2i + 1 is brought into the rotate-half order here: within
        # every head the even channels first, then the odd ones, for q and k alike (their products do not change), and
        # the per-head norm weights with them.
        D = spec.head_dim
        interleaved = spec.position is not None and getattr(spec.position, "pairing", "half") == "interleaved"
        order = torch.cat([torch.arange(0, D, 2), torch.arange(1, D, 2)]) if interleaved else None

        def per_head(t: torch.Tensor, heads: int) -> torch.Tensor:     # rows (or elements) of q or k, head by head
            if order is None:
                return t
            return t.reshape(heads, D, *t.shape[1:])[:, order].reshape(t.shape)

        wq, wk = per_head(weights[n["q"]], spec.heads), per_head(weights[n["k"]], spec.kv_heads)
        rows = [wq, wk, weights[n["v"]]]
        q_rows = [wq]
        biases = q_biases = None
        if spec.qkv_bias:
            bq = per_head(weights[n["q_bias"]], spec.heads)
            biases = [bq, per_head(weights[n["k_bias"]], spec.kv_heads), weights[n["v_bias"]]]
            q_biases = [bq]
        if spec.head_gate:
            g = weights[n["gate"]]
            pad = (-g.shape[0]) % 16      # (whole 16-row tiles: what the few-row product's unpredicated instances and its tails ask for)
            if pad:
                g = torch.cat([g, torch.zeros(pad, g.shape[1], dtype=g.dtype)], 0)
            rows.append(g)
            q_rows.append(g)
            if biases is not None:
                biases.append(torch.zeros(g.shape[0]))
                q_biases.append(torch.zeros(g.shape[0]))
        self.w_qkvg = rt.matrix(torch.cat([r.to(torch.float32) for r in rows], 0))
        self.b_qkvg = rt.vector(torch.cat([b.to(torch.float32) for b in biases])) if biases is not None else None
        self._q_rows, self._q_biases = q_rows, q_biases          # stacked on the device on the first use as a reader of another cache
        self.w_qg = self.b_qg = None
        self.w_o = rt.matrix(weights[n["o"]])
        self.q_norm = rt.vector(per_head(weights[n["q_norm"]], 1)) if spec.qk_norm else None
        self.k_norm = rt.vector(per_head(weights[n["k_norm"]], 1)) if spec.qk_norm else None
        self.position = (registry.position_class(spec.position.kind)(spec.position, rt)
                         if spec.position is not None else None)

    def takes_prenormed(self, rows: int) -> bool:
        return self.rt.few_rows_shape(rows, self.w_qkvg) and self.w_qkvg.shape[1] % 8 == 0

    def forward(self, x, step, cache, into=None) -> torch.Tensor:
        s, rt = self.spec, self.rt
        T = x.shape[0]
        if cache is None or cache.storage is None:
            raise RuntimeError("attention needs a key/value cache")
        if cache.owner:
            w_in, b_in, gate_at = self.w_qkvg, self.b_qkvg, self.q_dim + 2 * self.kv_dim
        else:
            if self.w_qg is None:
                self.w_qg = rt.matrix(torch.cat([r.to(torch.float32) for r in self._q_rows], 0))
                if self._q_biases is not None:
                    self.b_qg = rt.vector(torch.cat([b.to(torch.float32) for b in self._q_biases]))
            w_in, b_in, gate_at = self.w_qg, self.b_qg, self.q_dim
        table = step.page_tables[cache.group]
        rope = self.position.table(step.max_positions) if self.position is not None else None
        q = rt.ws.get("attn_q", (T, s.heads, s.head_dim), rt.act_dtype)
        if step.decode and rt.rope_behind_product(x, w_in, s.head_dim):
            # one token a sequence: the per-head norms, the rotation and the cache write run behind the product, in its kernel
            proj = rt.ws.get("attn_qkv", (T, w_in.shape[0]), rt.act_dtype)
            rt.few_rows_rope(x, w_in, proj, b_in, q_out=q, pool=cache.storage if cache.owner else None,
                             page_table=table if cache.owner else None, seq_of_token=step.seq_of_token,
                             positions=step.positions, q_w=self.q_norm, k_w=self.k_norm, rope=rope, heads=s.heads,
                             kv_heads=s.kv_heads, head_dim=s.head_dim, page_size=step.page_size, eps=s.qk_norm_eps)
        else:
            proj = rt.linear(x, w_in, "attn_qkv", b_in)
            ops.qk_norm_rope_store(proj, q, cache.storage, table, step.seq_of_token, step.positions, self.q_norm,
                                   self.k_norm, rope, s.heads, s.kv_heads, s.head_dim, step.page_size, s.qk_norm_eps,
                                   write_kv=cache.owner)
        o = rt.ws.get("attn_o", (T, s.heads, s.head_dim), rt.act_dtype)
        gate = proj[:, gate_at:] if s.head_gate else None
        self.attend(q, cache, table, step, gate, o)
        if into is not None:
            return into.product(o.view(T, self.q_dim), self.w_o)
        return rt.linear(o.view(T, self.q_dim), self.w_o, "mixer_out")

    def attend(self, q, cache, table, step, gate, o) -> None:
        s, rt = self.spec, self.rt
        if step.fixed_shape and rt.mode == "bfloat16" and ops.attention_mma_supports(s.head_dim, step.page_size, s.heads // s.kv_heads):
            # a step captured for any lengths up to its bounds: one key split, grids from the bounds
            if rt.prompt_attention == "tcgen05" and ops.attention_tc_supports(s.head_dim, step.page_size, s.heads // s.kv_heads):
                ops.attention_tc(q, cache.storage, table, step.cu_seqlens, step.kv_lens, gate, o, step.n_seqs,
                                 step.max_q_len, s.kv_heads, step.page_size, s.scale, s.window, step.max_kv_len)
            else:
                ops.attention_mma(q, cache.storage, table, step.cu_seqlens, step.kv_lens, gate, o, None, step.n_seqs,
                                  step.max_q_len, s.kv_heads, step.page_size, s.scale, s.window, 1)
            return
        if rt.mode == "bfloat16" and ops.attention_mma_supports(s.head_dim, step.page_size, s.heads // s.kv_heads):
            # Few tiles and long key ranges (decoding): split each range over several CTAs so that
            # every SM streams a part of the cache; the partial results meet in scratch memory.
            tokens_per_tile = 64 // (s.heads // s.kv_heads)
            tiles = sum(-(-int(n) // tokens_per_tile) for n in step.q_lens_host) * s.kv_heads
            blocks = -(-step.max_kv_len // step.page_size)
            if s.window > 0:
                blocks = min(blocks, -(-(s.window + step.max_q_len) // step.page_size) + 1)
            if step.decode and s.heads // s.kv_heads <= 16 and rt.attn_split_factor == 0:
                splits = decode_splits(tiles, blocks, max(1, ops.attention_mma_decode_slots(s.head_dim, tiles)),
                                       rt.attn_fixed_cost)
            else:
                splits = max(1, min(blocks, 32, (max(rt.attn_split_factor, 1) * rt.sm_count) // max(tiles, 1)))
            # prompts: the tcgen05 kernel, unless few tiles face many keys (a short piece of a long sequence), where
            # cutting the keys over more CTAs is worth more
            if ((splits == 1 or step.max_kv_len <= 512) and not step.decode and rt.prompt_attention == "tcgen05"
                    and ops.attention_tc_supports(s.head_dim, step.page_size, s.heads // s.kv_heads)):
                ops.attention_tc(q, cache.storage, table, step.cu_seqlens, step.kv_lens, gate, o, step.n_seqs,
                                 step.max_q_len, s.kv_heads, step.page_size, s.scale, s.window, step.max_kv_len)
                return
            scratch = None
            if splits > 1:
                need = ops.attention_mma_scratch_bytes(q.shape[0] * s.heads, s.head_dim, splits)
                scratch = rt.ws.get("attn_scratch", (need,), torch.uint8)
            counters = rt.attn_counters if (rt.fuse_tails and rt.tail_attn and step.n_seqs * s.kv_heads <= rt.attn_counters.numel()) else None
            ops.attention_mma(q, cache.storage, table, step.cu_seqlens, step.kv_lens, gate, o, scratch, step.n_seqs,
                              step.max_q_len, s.kv_heads, step.page_size, s.scale, s.window, splits, counters=counters,
                              bounded_waits=step.decode)
            return
        ops.attention_generic(q, cache.storage, table, step.seq_of_token, step.positions, gate, o, s.kv_heads,
                              step.page_size, s.scale, s.window)


registry.register_mixer(AttentionMixer.kind, AttentionMixer)
