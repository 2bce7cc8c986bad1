"""Loads the compiled CUDA library and calls its `extern "C"` functions on torch tensors.

There is no fallback: if the library cannot be built or loaded, or a function reports an
error, an exception says so. Tensors are passed as raw device pointers with their sizes;
launches go to torch's current CUDA stream, so they order with torch's own work and can
be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_lib = None
launches = 0      # kernels launched through this module since import (a graph replay counts its kernels too)


def _signatures(lib) -> None:
    P, I, L, F = c_void_p, c_int, c_int64, c_float
    sig = {
        "xs_embed": [P, I, P, P, I, I, F, P],
        "xs_logit_cap": [P, L, F, P],
        "xs_add_rmsnorm": [P, P, I, P, P, P, I, P, I, I, F, F, P],
        "xs_silu_mul": [P, P, I, I, I, L, I, P],
        "xs_zero_rows": [P, P, I, L, P],
        "xs_gemm_generic": [P, P, P, P, I, I, I, I, I, L, L, L, P],
        "xs_qk_norm_rope_store": [P, L, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P],
        "xs_attention_generic": [P, P, P, I, P, P, P, L, P, I, I, I, I, I, F, I, I, P],
        "xs_short_conv": [P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
        "xs_attention_mma": [P, P, P, I, P, P, P, L, P, P, L, I, I, I, I, I, I, I, F, I, I, P],
        "xs_attention_tc": [P, P, L, P, I, P, P, P, L, P, I, I, I, I, I, I, I, F, I, I, P, P],
        "xs_gemm_small_m": [P, P, P, P, P, I, I, I, I, L, L, L, I, I, P, L, P],
        "xs_gemm_small_m_normed": [P, P, P, P, P, I, I, I, I, L, L, L, I, I, P, L, P, I, I, F, P, P, L, P, P],
        "xs_gemm_small_m_ex": [P, P, P, P, P, I, I, I, I, L, L, L, I, I, P, L, P, I, I, F, P, P, L, P,
                               P, P, P, P, P, P, I, I, P, P, P, P],
        "xs_gemm_small_m_rope": [P, P, P, P, I, I, I, L, L, L, P, I, I, F, P, P, P, I, P, P, P, P, P, I, I, I, I, F, P],
        "xs_attention_mma_merged": [P, P, P, I, P, P, P, L, P, P, L, P, L, P, I, I, I, I, I, I, I, F, I, I, P],
        "xs_gemm_tc": [P, P, P, P, I, I, I, I, I, L, L, L, I, P, L, P, P],
        "xs_argmax": [P, L, I, I, P, P, P],
        "xs_sample": [P, L, I, I, P, P, P, P, P, P, I, P, P],
        "xs_apply_penalties": [P, L, I, I, P, P, P, P, P, P, P],
        "xs_note_tokens": [P, P, I, I, P, P, I, P],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    lib.xs_last_error.restype = ctypes.c_char_p
    lib.xs_last_error.argtypes = []
    lib.xs_uniform.restype = c_double
    lib.xs_uniform.argtypes = [c_uint64, c_uint64]
    lib.xs_abi_version.restype = c_int
    lib.xs_attention_mma_scratch_bytes.restype = c_int64
    lib.xs_attention_mma_scratch_bytes.argtypes = [c_int64, c_int, c_int]
    lib.xs_attention_mma_supports.restype = c_int
    lib.xs_attention_mma_supports.argtypes = [c_int, c_int, c_int]
    lib.xs_attention_tc_supports.restype = c_int
    lib.xs_attention_tc_supports.argtypes = [c_int, c_int, c_int]
    lib.xs_attention_mma_decode_slots.restype = c_int
    lib.xs_attention_mma_decode_slots.argtypes = [c_int, c_int64]
    lib.xs_gemm_small_m_supports.restype = c_int
    lib.xs_gemm_small_m_supports.argtypes = [c_int, c_int, c_int64, c_int64]
    lib.xs_gemm_tc_supports.restype = c_int
    lib.xs_gemm_tc_supports.argtypes = [c_int, c_int, c_int, c_int64, c_int64]
    lib.xs_gemm_tc_tile_n.restype = c_int
    lib.xs_gemm_tc_tile_n.argtypes = [c_int]
    lib.xs_gemm_tc_scratch_bytes.restype = c_int64
    lib.xs_gemm_tc_scratch_bytes.argtypes = [c_int, c_int, c_int]
    lib.xs_gemm_small_m_ksplit.restype = c_int
    lib.xs_gemm_small_m_ksplit.argtypes = [c_int, c_int, c_int, c_int]
    lib.xs_gemm_small_m_scratch_bytes.restype = c_int64
    lib.xs_gemm_small_m_scratch_bytes.argtypes = [c_int, c_int, c_int]


class _Watched:
    """The library behind two debugging switches (the reference has the same pair for its own backend,
    XS_SYCL_PROFILE and XS_SYCL_SYNC, src/backend/sycl/sycl_backend.cpp:351-353, 2520-2570):

    XS_PROFILE=1  CUDA events around every launch; `profile_report()` (also printed at exit) sums the device time by
                  kernel function and by its sizes (the call's integer arguments).
    XS_SYNC=1     the device is waited for after every launch, and an error that shows up there is raised with the
                  name and the sizes of the launch it belongs to, instead of surfacing at some later call.

    Both run every step kernel by kernel (no CUDA graphs: engine/model.py) and cost time; neither is on by default."""

    def __init__(self, lib, profile: bool, sync: bool):
        self._lib, self._profile, self._sync = lib, profile, sync
        self.spans = []         # (name, sizes, start event, end event)
        self._name = lib._name

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        argtypes = getattr(fn, "argtypes", None)
        if not name.startswith("xs_") or not argtypes or argtypes[-1] is not c_void_p or fn.restype is not c_int:
            return fn           # not a launch (a query, a switch)

        def call(*args):
            sizes = tuple(a for a, t in zip(args, argtypes) if t in (c_int, c_int64) and isinstance(a, int) and abs(a) < (1 << 40))
            capturing = torch.cuda.is_current_stream_capturing()
            if self._profile and not capturing:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                rc = fn(*args)
                end.record()
                self.spans.append((name, sizes, start, end))
            else:
                rc = fn(*args)
            if self._sync and not capturing and rc == 0:
                try:
                    torch.cuda.synchronize()
                except RuntimeError as e:
                    raise KernelError(f"{name}{sizes}: the device reported an error after this launch: {e}") from None
            return rc

        call.__name__ = name
        setattr(self, name, call)
        return call


def profile_report(reset: bool = True, file=None) -> dict:
    """{(kernel function, sizes): (launches, total microseconds)} of the launches made under XS_PROFILE=1 since
    the last report, printed as a table (largest first) to `file` (standard error)."""
    import sys
    lib = _lib
    if not isinstance(lib, _Watched) or not lib.spans:
        return {}
    torch.cuda.synchronize()
    table = {}
    for name, sizes, start, end in lib.spans:
        n, us = table.get((name, sizes), (0, 0.0))
        table[(name, sizes)] = (n + 1, us + start.elapsed_time(end) * 1e3)
    if reset:
        lib.spans = []
    out = file or sys.stderr
    total = sum(us for _, us in table.values())
    print(f"[xpu_serve_b200 profile] {sum(n for n, _ in table.values())} launches, {total:.0f} us on the device", file=out)
    for (name, sizes), (n, us) in sorted(table.items(), key=lambda kv: -kv[1][1]):
        print(f"  {us:10.1f} us {100 * us / max(total, 1e-9):5.1f} %  x{n:<5d} {name} {sizes}", file=out)
    return table


def load(verbose: bool = True):
    """The library handle, built first if its file is missing."""
    global _lib
    if _lib is None:
        path = _build.build(verbose=verbose)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the CUDA library {path} cannot be loaded: {e}") from None
        _signatures(lib)
        # tuning switches, read once (defaults are what measured best on B200)
        if "XS_ATTN_DECODE_STAGES" in os.environ:
            lib.xs_attention_mma_set_decode_stages(int(os.environ["XS_ATTN_DECODE_STAGES"]))
        if os.environ.get("XS_NO_ONE_ROUND", "0") == "1":
            lib.xs_gemm_small_m_set_one_round(0)
        if "XS_ATTN_PREFETCH_BLOCKS" in os.environ:
            lib.xs_attention_mma_set_prefetch_blocks(int(os.environ["XS_ATTN_PREFETCH_BLOCKS"]))
        if os.environ.get("XS_NO_PDL", "0") == "1":
            lib.xs_set_pdl(0)
        if os.environ.get("XS_TC_NO_PAIR", "0") == "1":
            lib.xs_gemm_tc_set_pair(0)
        if "XS_ATTN_TMA_CARVEOUT" in os.environ:
            lib.xs_attention_mma_set_tma_carveout(int(os.environ["XS_ATTN_TMA_CARVEOUT"]))
        if "XS_ATTN_DECODE_TMA" in os.environ:        # "0": cp.async kernel for every head size; "n" (2..6): that many stages
            n = int(os.environ["XS_ATTN_DECODE_TMA"])
            lib.xs_attention_mma_set_decode_tma(1 if n > 0 else 0, n)
        profile, sync = os.environ.get("XS_PROFILE", "0") == "1", os.environ.get("XS_SYNC", "0") == "1"
        if profile or sync:
            lib = _Watched(lib, profile, sync)
            if profile:
                import atexit
                atexit.register(profile_report)
        _lib = lib
    return _lib


def watched() -> bool:
    """Whether XS_PROFILE or XS_SYNC is on (steps then run kernel by kernel, without CUDA graphs)."""
    return os.environ.get("XS_PROFILE", "0") == "1" or os.environ.get("XS_SYNC", "0") == "1"


def loaded_path() -> Optional[str]:
    return None if _lib is None else _lib._name


def _check(rc: int, kernels: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(_lib.xs_last_error().decode("utf-8", "replace"))
    launches += kernels


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (inside a graph capture: the capturing stream). Asked of torch's C layer directly
    where it offers that: `torch.cuda.current_stream()` builds a Python object per call, a hundred times a step."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32, bfloat16 are)") from None


def _need(t: torch.Tensor, what: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def uniform(seed: int, counter: int) -> float:
    """The uniform in [0, 1) that the sampling kernel derives from (seed, counter)."""
    return float(load().xs_uniform(seed & (2 ** 64 - 1), counter & (2 ** 64 - 1)))


# ------------------------------------------------------------------ wrappers
def embed(table: torch.Tensor, ids: torch.Tensor, h: torch.Tensor, scale: float = 1.0) -> None:
    """h[t] = table[ids[t]] * scale, float32."""
    _need(table, "embedding table"); _need(ids, "ids", torch.int32); _need(h, "h", torch.float32)
    T, H = h.shape
    _check(load().xs_embed(table.data_ptr(), _code(table), ids.data_ptr(), h.data_ptr(), T, H, float(scale), _stream()))


def logit_cap(logits: torch.Tensor, cap: float) -> None:
    """logits = cap * tanh(logits / cap), in place."""
    _need(logits, "logits", torch.float32)
    _check(load().xs_logit_cap(logits.data_ptr(), logits.numel(), float(cap), _stream()))


def add_rmsnorm(h: torch.Tensor, m: Optional[torch.Tensor], post_w: Optional[torch.Tensor],
                w: Optional[torch.Tensor], y: Optional[torch.Tensor], rows: Optional[torch.Tensor], eps: float,
                eps_post: Optional[float] = None) -> None:
    """h += post(m) (if m); y = RMSNorm(h, w) (if w), over `rows` of h when given."""
    _need(h, "h", torch.float32)
    H = h.shape[-1]
    n = h.shape[0] if rows is None else rows.numel()
    if m is not None:
        _need(m, "m")
        if m.shape != h.shape:
            raise KernelError(f"m is {tuple(m.shape)}, h is {tuple(h.shape)}")
    for v, name in ((post_w, "post_w"), (w, "w")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != H:
                raise KernelError(f"{name} has {v.numel()} elements for rows of {H}")
    if y is not None:
        _need(y, "y")
        if y.shape[0] < n or y.shape[-1] != H:
            raise KernelError(f"y is {tuple(y.shape)} for {n} rows of {H}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _check(load().xs_add_rmsnorm(h.data_ptr(), _ptr(m), F32 if m is None else _code(m), _ptr(post_w), _ptr(w),
                                 _ptr(y), F32 if y is None else _code(y), _ptr(rows), n, H,
                                 float(eps if eps_post is None else eps_post), float(eps), _stream()))


def silu_mul(gu: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
    """out = silu(gate) * up. interleave 0: a row of gu is [gate | up]; 8: blocks of 8 gate, 8 up columns."""
    _need(out, "out", gu.dtype)
    if not gu.is_cuda or gu.dim() != 2 or gu.stride(1) != 1:
        raise KernelError("gate_up must be a CUDA matrix with contiguous rows")
    T, F = out.shape
    if gu.shape[0] != T or gu.shape[1] < 2 * F:
        raise KernelError(f"gate_up is {tuple(gu.shape)} for an output of {tuple(out.shape)}")
    _check(load().xs_silu_mul(gu.data_ptr(), out.data_ptr(), _code(gu), T, F, gu.stride(0), int(interleave), _stream()))


def zero_rows(state: torch.Tensor, slots: torch.Tensor) -> None:
    _need(state, "state"); _need(slots, "slots", torch.int32)
    row_bytes = state[0].numel() * state.element_size()
    _check(load().xs_zero_rows(state.data_ptr(), slots.data_ptr(), slots.numel(), row_bytes, _stream()))


def gemm_generic(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T (+ bias). Rows may be strided; columns are contiguous."""
    for t, name in ((x, "x"), (w, "w"), (out, "out")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm: {name} must be a CUDA matrix with contiguous rows")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or x.dtype != w.dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    _check(load().xs_gemm_generic(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), _code(x), _code(out),
                                  M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()))


def qk_norm_rope_store(qkv: torch.Tensor, q_out: torch.Tensor, pool: Optional[torch.Tensor],
                       page_table: Optional[torch.Tensor], seq_of_token: torch.Tensor, positions: torch.Tensor,
                       q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], rope: Optional[torch.Tensor],
                       heads: int, kv_heads: int, head_dim: int, page_size: int, eps: float, write_kv: bool) -> None:
    _need(q_out, "q_out", qkv.dtype)
    if qkv.stride(1) != 1:
        raise KernelError("qkv rows must be contiguous")
    T = qkv.shape[0]
    width = (heads + (2 * kv_heads if write_kv else 0)) * head_dim
    if qkv.shape[1] < width:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, needs {width} columns")
    if write_kv:
        _need(pool, "cache", qkv.dtype); _need(page_table, "page table", torch.int32)
        if tuple(pool.shape[1:]) != (2, kv_heads, page_size, head_dim):
            raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {head_dim}]")
    for v, name in ((q_w, "q_norm"), (k_w, "k_norm")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != head_dim:
                raise KernelError(f"{name} has {v.numel()} elements for heads of {head_dim}")
    if rope is not None:
        _need(rope, "rope table", torch.float32)
        if tuple(rope.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"rope table is {tuple(rope.shape)}, expected [*, {head_dim // 2}, 2]")
    P = 0 if page_table is None else page_table.shape[1]
    _check(load().xs_qk_norm_rope_store(
        qkv.data_ptr(), qkv.stride(0), q_out.data_ptr(), _ptr(pool), _ptr(page_table), P, seq_of_token.data_ptr(),
        positions.data_ptr(), _ptr(q_w), _ptr(k_w), _ptr(rope), T, heads, kv_heads, head_dim, page_size, float(eps),
        1 if write_kv else 0, _code(qkv), _stream()))


def attention_generic(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, seq_of_token: torch.Tensor,
                      positions: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, kv_heads: int,
                      page_size: int, scale: float, window: int) -> None:
    _need(q, "q"); _need(out, "out", q.dtype); _need(pool, "cache", q.dtype); _need(page_table, "page table", torch.int32)
    T, heads, D = q.shape
    if tuple(pool.shape[1:]) != (2, kv_heads, page_size, D):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {D}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < heads:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {heads} heads")
        ld_gate = gate.stride(0)
    _check(load().xs_attention_generic(
        q.data_ptr(), pool.data_ptr(), page_table.data_ptr(), page_table.shape[1], seq_of_token.data_ptr(),
        positions.data_ptr(), _ptr(gate), ld_gate, out.data_ptr(), T, heads, kv_heads, D, page_size, float(scale),
        int(window), _code(q), _stream()))


def attention_mma_supports(head_dim: int, page_size: int, group: int) -> bool:
    return bool(load().xs_attention_mma_supports(head_dim, page_size, group))


def attention_mma_decode_slots(head_dim: int, tiles: int) -> int:
    """CTAs of the decode attention kernel that run at one time on the device when `tiles` = sequences x kv heads
    (the kernel keeps fewer stages, and so more CTAs an SM, when the tiles alone overfill the device)."""
    return int(load().xs_attention_mma_decode_slots(head_dim, tiles))


def attention_mma_scratch_bytes(rows: int, head_dim: int, splits: int) -> int:
    return int(load().xs_attention_mma_scratch_bytes(rows, head_dim, splits))


def attention_mma(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, cu_seqlens: torch.Tensor,
                  kv_lens: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor,
                  scratch: Optional[torch.Tensor], n_seqs: int, max_q_len: int, kv_heads: int, page_size: int,
                  scale: float, window: int, splits: int, counters: Optional[torch.Tensor] = None,
                  bounded_waits: bool = False) -> None:
    """Tensor-core attention over the paged bfloat16 cache. `scratch`: a byte buffer of at least
    attention_mma_scratch_bytes(tokens * heads, head_dim, splits) when splits > 1. `counters`: at least
    n_seqs * kv_heads zeroed int32 words that the kernel leaves zeroed; with them a decode step (one token a
    sequence) merges its key splits inside the attention kernel instead of in a second one. `bounded_waits`: a decode
    step at head size 64 may take the kernel that the TMA unit feeds; its waits are bounded, and one that gives up sets
    gemm_tc_status(device), which the caller then has to look at (tc_status_unread)."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pool, "cache", torch.bfloat16)
    _need(page_table, "page table", torch.int32)
    T, heads, D = q.shape
    if tuple(pool.shape[1:]) != (2, kv_heads, page_size, D):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {D}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < heads:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {heads} heads")
        ld_gate = gate.stride(0)
    sbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    merged = counters is not None and splits > 1 and max_q_len == 1 and heads // kv_heads <= 16
    if merged:
        _need(counters, "counters", torch.int32)
        if counters.numel() < n_seqs * kv_heads:
            raise KernelError(f"attention: {counters.numel()} counters for {n_seqs} sequences of {kv_heads} kv heads")
    tma = bounded_waits and max_q_len == 1 and D == 64 and heads // kv_heads <= 16
    if tma:
        mark_bounded(q.device)
    _check(load().xs_attention_mma_merged(
        q.data_ptr(), pool.data_ptr(), page_table.data_ptr(), page_table.shape[1], cu_seqlens.data_ptr(),
        kv_lens.data_ptr(), _ptr(gate), ld_gate, out.data_ptr(), _ptr(scratch), sbytes, _ptr(counters) if merged else None,
        pool.shape[0] if tma else 0, gemm_tc_status(q.device).data_ptr() if tma else None,
        T, n_seqs, max_q_len, heads, kv_heads, D, page_size, float(scale), int(window), int(splits), _stream()),
        kernels=2 if splits > 1 and not merged else 1)


def attention_tc_supports(head_dim: int, page_size: int, group: int) -> bool:
    return bool(load().xs_attention_tc_supports(head_dim, page_size, group))


def attention_tc(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, cu_seqlens: torch.Tensor,
                 kv_lens: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, n_seqs: int, max_q_len: int,
                 kv_heads: int, page_size: int, scale: float, window: int, max_kv_len: int = 0) -> None:
    """Attention for prompts on the tcgen05 tensor cores (head size 64): the same operation as attention_mma with
    one key split. A wait that gives up inside the kernel sets gemm_tc_status(device). `max_kv_len` (the longest
    sequence's keys, 0 if unknown) only picks the order in which the kernel's CTAs start."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pool, "cache", torch.bfloat16)
    _need(page_table, "page table", torch.int32)
    T, heads, D = q.shape
    if tuple(pool.shape[1:]) != (2, kv_heads, page_size, D):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {D}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < heads:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {heads} heads")
        ld_gate = gate.stride(0)
    mark_bounded(q.device)
    _check(load().xs_attention_tc(
        q.data_ptr(), pool.data_ptr(), pool.shape[0], page_table.data_ptr(), page_table.shape[1], cu_seqlens.data_ptr(),
        kv_lens.data_ptr(), _ptr(gate), ld_gate, out.data_ptr(), T, n_seqs, max_q_len, heads, kv_heads, D, page_size,
        float(scale), int(window), int(max_kv_len), gemm_tc_status(q.device).data_ptr(), _stream()))


def gemm_small_m_supports(M: int, K: int, ldx: int, ldw: int) -> bool:
    return bool(load().xs_gemm_small_m_supports(M, K, ldx, ldw))


def gemm_small_m_ksplit(M: int, N: int, K: int, sms: int) -> int:
    """The number of K slices the kernel prefers for this shape on a device with `sms` SMs."""
    return int(load().xs_gemm_small_m_ksplit(M, N, K, sms))


def gemm_small_m_scratch_bytes(M: int, N: int, ksplit: int) -> int:
    return int(load().xs_gemm_small_m_scratch_bytes(M, N, ksplit))


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, swiglu: bool = False, ksplit: int = 1,
                 scratch: Optional[torch.Tensor] = None, in_ssq: Optional[torch.Tensor] = None, in_width: int = 0,
                 in_eps: float = 0.0, next_w: Optional[torch.Tensor] = None, next_x: Optional[torch.Tensor] = None,
                 out_ssq: Optional[torch.Tensor] = None, conv: Optional[dict] = None,
                 argmax: Optional[tuple] = None) -> None:
    """out[M, N] = x . w^T (+ bias) for M <= 16, bfloat16 operands; or residual (float32) += the product;
    or, with swiglu, out[M, N / 2] = silu(gate) * up for a weight stacked as blocks of 8 gate and 8 up rows.
    ksplit > 1 cuts K over several CTAs; `scratch` is then a zero-initialised byte buffer of at least
    gemm_small_m_scratch_bytes, kept (whole) from call to call.

    RMSNorm across the product: with `residual`, `next_w` [N] and `next_x` [M, N] bfloat16, the kernel also
    leaves next_x = bfloat16(residual * next_w) and, in `out_ssq` [ceil(N / 16), 16] float32, each tile's
    sums of squares of the new residual values per row. A product given that `out_ssq` as `in_ssq` (with the
    residual's width and the norm's eps) and that `next_x` as x scales its result by each row's
    1 / sqrt(mean square + eps): together they are norm(residual) . w^T without a norm kernel between.

    Work behind the product, in the same kernel: `conv` = dict(taps [k, H] float32, bias [H] or None, state
    [slots, k - 1, H] bfloat16, slots [M] int32, out [M, H] bfloat16, counters: H / 16 zeroed int32 words, left
    zeroed): the product is a short-convolution layer's in_proj for one token a sequence, out = [B | C | X], and the
    gated convolution with its state update follows. `argmax` = (out [M] int32, keys: 16 zeroed int64 words,
    counter: one zeroed int32 word; both left zeroed): each row's column of the largest output."""
    for t, name in ((x, "x"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
            raise KernelError(f"gemm (few rows): {name} must be a bfloat16 CUDA matrix with contiguous rows")
    M, K = x.shape
    N = w.shape[0]
    target = residual if residual is not None else out
    if w.shape[1] != K or target is None or tuple(target.shape) != (M, N // 2 if swiglu else N) or target.stride(1) != 1:
        raise KernelError(f"gemm (few rows): x {tuple(x.shape)}, w {tuple(w.shape)}, out "
                          f"{None if target is None else tuple(target.shape)}")
    if residual is not None and residual.dtype != torch.float32:
        raise KernelError("gemm (few rows): the residual must be float32")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    in_tiles = 0
    if in_ssq is not None:
        _need(in_ssq, "in_ssq", torch.float32)
        if in_ssq.dim() != 2 or in_ssq.shape[1] != 16 or not in_ssq.is_contiguous() or in_width <= 0:
            raise KernelError(f"gemm (few rows): sums of squares {tuple(in_ssq.shape)} over a width of {in_width}")
        in_tiles = in_ssq.shape[0]
    ld_next = 0
    if next_x is not None or next_w is not None or out_ssq is not None:
        if next_x is not None:
            _need(next_w, "next_w", torch.float32); _need(next_x, "next_x", torch.bfloat16)
            if tuple(next_x.shape) != (M, N) or next_x.stride(1) != 1 or next_w.numel() != N or not next_w.is_contiguous():
                raise KernelError(f"gemm (few rows): next_x {tuple(next_x.shape)}, next_w {tuple(next_w.shape)} for [{M}, {N}]")
            ld_next = next_x.stride(0)
        _need(out_ssq, "out_ssq", torch.float32)
        if tuple(out_ssq.shape) != ((N + 15) // 16, 16) or not out_ssq.is_contiguous():
            raise KernelError(f"gemm (few rows): out_ssq is {tuple(out_ssq.shape)}, expected [{(N + 15) // 16}, 16]")
    cv = [None] * 6 + [0, 0]
    if conv is not None:
        taps, state, slots, cout, counters = conv["taps"], conv["state"], conv["slots"], conv["out"], conv["counters"]
        k, H = taps.shape
        _need(taps, "taps", torch.float32); _need(state, "state", torch.bfloat16); _need(slots, "slots", torch.int32)
        _need(cout, "conv out", torch.bfloat16); _need(counters, "conv counters", torch.int32)
        if conv.get("bias") is not None:
            _need(conv["bias"], "conv bias", torch.float32)
        if (N != 3 * H or tuple(state.shape[1:]) != (k - 1, H) or slots.numel() < M or tuple(cout.shape) != (M, H)
                or counters.numel() < H // 16 or out is None or out.dtype != torch.bfloat16):
            raise KernelError(f"gemm (few rows): convolution of {k} taps over {H} channels behind a product of {N} columns, "
                              f"state {tuple(state.shape)}, out {tuple(cout.shape)}")
        cv = [taps.data_ptr(), _ptr(conv.get("bias")), state.data_ptr(), slots.data_ptr(), cout.data_ptr(),
              counters.data_ptr(), int(k), int(H)]
    am = [None, None, None]
    if argmax is not None:
        a_out, keys, counter = argmax
        _need(a_out, "argmax out", torch.int32); _need(keys, "argmax keys", torch.int64); _need(counter, "argmax counter", torch.int32)
        if a_out.numel() < M or keys.numel() < 16 or M > 16:
            raise KernelError(f"gemm (few rows): argmax of {M} rows into {a_out.numel()} words")
        am = [keys.data_ptr(), counter.data_ptr(), a_out.data_ptr()]
    _check(load().xs_gemm_small_m_ex(
        x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(out), _ptr(residual), F32 if out is None else _code(out), M, N, K,
        x.stride(0), w.stride(0), target.stride(0), 1 if swiglu else 0, int(ksplit), _ptr(scratch),
        0 if scratch is None else scratch.numel() * scratch.element_size(), _ptr(in_ssq), in_tiles, int(in_width),
        float(in_eps), _ptr(next_w), _ptr(next_x), ld_next, _ptr(out_ssq), *cv, *am, _stream()))


def gemm_small_m_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor],
                      q_out: torch.Tensor, pool: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                      seq_of_token: torch.Tensor, positions: torch.Tensor, q_w: Optional[torch.Tensor],
                      k_w: Optional[torch.Tensor], rope: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int,
                      page_size: int, eps: float, in_ssq: Optional[torch.Tensor] = None, in_width: int = 0,
                      in_eps: float = 0.0) -> None:
    """An attention layer's q/k/v product for one token a sequence (M <= 16, bfloat16) with what qk_norm_rope_store does
    behind it in the same kernel: out [M, N] = x . w^T (+ bias) as gemm_small_m leaves it (its columns behind the heads,
    the head gate's, are what the caller still reads), and from its columns (heads x head_dim of q, then, with `pool`,
    kv_heads x head_dim of k and of v): per-head RMSNorm (q_w, k_w), rotation by `rope` [positions, head_dim / 2, 2],
    queries to q_out [M, heads, head_dim], keys and raw values into the cache's pages. Head sizes 32, 64, 128."""
    for t, name in ((x, "x"), (w, "w"), (out, "out"), (q_out, "q_out")):
        _need(t, name, torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    width = (heads + (2 * kv_heads if pool is not None else 0)) * head_dim
    if (x.stride(1) != 1 or w.stride(1) != 1 or w.shape[1] != K or tuple(out.shape) != (M, N) or out.stride(1) != 1
            or N < width or tuple(q_out.shape) != (M, heads, head_dim) or not q_out.is_contiguous()
            or head_dim not in (32, 64, 128) or M > 16):
        raise KernelError(f"gemm (few rows) with rotation: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"q_out {tuple(q_out.shape)}, {heads} + 2 x {kv_heads} heads of {head_dim}")
    _need(seq_of_token, "seq_of_token", torch.int32); _need(positions, "positions", torch.int32)
    if seq_of_token.numel() < M or positions.numel() < M:
        raise KernelError("gemm (few rows) with rotation: a sequence and a position per row")
    P_ = 0
    if pool is not None:
        _need(pool, "cache", torch.bfloat16); _need(page_table, "page table", torch.int32)
        if tuple(pool.shape[1:]) != (2, kv_heads, page_size, head_dim):
            raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {head_dim}]")
        P_ = page_table.shape[1]
    for v, name in ((q_w, "q_norm"), (k_w, "k_norm")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != head_dim:
                raise KernelError(f"{name} has {v.numel()} elements for heads of {head_dim}")
    if rope is not None:
        _need(rope, "rope table", torch.float32)
        if tuple(rope.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"rope table is {tuple(rope.shape)}, expected [*, {head_dim // 2}, 2]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    in_tiles = 0
    if in_ssq is not None:
        _need(in_ssq, "in_ssq", torch.float32)
        if in_ssq.dim() != 2 or in_ssq.shape[1] != 16 or not in_ssq.is_contiguous() or in_width <= 0:
            raise KernelError(f"gemm (few rows): sums of squares {tuple(in_ssq.shape)} over a width of {in_width}")
        in_tiles = in_ssq.shape[0]
    _check(load().xs_gemm_small_m_rope(
        x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), out.stride(0),
        _ptr(in_ssq), in_tiles, int(in_width), float(in_eps), q_out.data_ptr(), _ptr(pool), _ptr(page_table), P_,
        seq_of_token.data_ptr(), positions.data_ptr(), _ptr(q_w), _ptr(k_w), _ptr(rope), heads, kv_heads, head_dim,
        page_size, float(eps), _stream()))


EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
_tc_status = {}


def gemm_tc_supports(T: int, N: int, K: int, ldx: int, ldw: int) -> bool:
    return bool(load().xs_gemm_tc_supports(T, N, K, ldx, ldw))


def gemm_tc_scratch_bytes(T: int, N: int, ksplit: int) -> int:
    return int(load().xs_gemm_tc_scratch_bytes(T, N, ksplit))


def gemm_tc_status(device) -> torch.Tensor:
    """The device word that the tcgen05 kernels set non-zero when one of their waits gave up."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _tc_status:
        _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[device]


# Devices on which a kernel with bounded waits (the tcgen05 kernels, decode attention fed by the TMA unit) was launched
# since the status word was last looked at. Whoever next waits for the device anyway (the generation loop for its
# tokens, trace replay for its logits) reads the word with what it waits for and hands it to `tc_status_read`.
_tc_unread = set()


bounded_launches = 0      # launches of kernels with bounded waits since import (a graph's capture counts its own)


def mark_bounded(device) -> None:
    """A kernel with bounded waits was launched (or a graph that holds one replayed) on `device`."""
    global bounded_launches
    bounded_launches += 1
    _tc_unread.add(gemm_tc_status(device).device)


def tc_status_unread(device) -> bool:
    return gemm_tc_status(device).device in _tc_unread


def tc_status_read(value: int, device) -> None:
    """`value`: the status word as copied from the device after every tcgen05 kernel launched so far has run.
    Non-zero: a bounded wait inside such a kernel gave up, so what the step wrote (activations, keys and
    values in the cache) is partly computed: the word is cleared and the step fails."""
    word = gemm_tc_status(device)
    _tc_unread.discard(word.device)
    if int(value) != 0:
        word.zero_()
        raise KernelError(f"a tcgen05 kernel gave up waiting (status {int(value)}): this step's results and what it "
                          f"wrote to the cache are not valid")


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            epilogue: int = EPI_STORE, ksplit: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """x[T, K] . w[N, K]^T on tcgen05 tensor cores (bfloat16 operands). epilogue EPI_STORE: out[T, N] bfloat16 or
    float32; EPI_RESIDUAL: out float32 += product; EPI_SWIGLU: out[T, N / 2] = silu(gate) * up for a weight stacked
    in blocks of 8 gate and 8 up rows."""
    for t, name in ((x, "x"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
            raise KernelError(f"gemm (tcgen05): {name} must be a bfloat16 CUDA matrix with contiguous rows")
    T, K = x.shape
    N = w.shape[0]
    cols = N // 2 if epilogue == EPI_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (T, cols) or out.stride(1) != 1:
        raise KernelError(f"gemm (tcgen05): x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    mark_bounded(x.device)
    _check(load().xs_gemm_tc(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), _code(out), int(epilogue), T, N, K,
                             x.stride(0), w.stride(0), out.stride(0), int(ksplit), _ptr(scratch),
                             0 if scratch is None else scratch.numel() * scratch.element_size(),
                             gemm_tc_status(x.device).data_ptr(), _stream()))


def short_conv(bcx: torch.Tensor, w_t: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
               all_single: bool = False) -> None:
    """`all_single`: every sequence brings exactly one token (lets one kernel also move the state)."""
    _need(out, "out", bcx.dtype); _need(state, "state", bcx.dtype); _need(w_t, "taps", torch.float32)
    T, H = out.shape
    K = w_t.shape[0]
    if bcx.stride(1) != 1 or bcx.shape[0] != T or bcx.shape[1] < 3 * H or w_t.shape[1] != H:
        raise KernelError(f"short_conv: bcx {tuple(bcx.shape)}, taps {tuple(w_t.shape)}, out {tuple(out.shape)}")
    if tuple(state.shape[1:]) != (K - 1, H):
        raise KernelError(f"short_conv: state is {tuple(state.shape)}, expected [*, {K - 1}, {H}]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    _check(load().xs_short_conv(bcx.data_ptr(), bcx.stride(0), w_t.data_ptr(), _ptr(bias), state.data_ptr(),
                                seq_of_token.data_ptr(), cu_seqlens.data_ptr(), slots.data_ptr(), out.data_ptr(),
                                T, slots.numel(), H, K, _code(bcx), 1 if all_single else 0, _stream()),
           kernels=1 if all_single and bcx.dtype == torch.bfloat16 and H % 8 == 0 and K <= 8 else 2)


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = index of the largest of row i, the lowest index among equals."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    n, V = logits.shape
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch.numel() < n:       # zeroed words the wide-row path works in and leaves zeroed
        scratch = _argmax_scratch[logits.device] = torch.zeros(max(n, 256), dtype=torch.int64, device=logits.device)
    _check(load().xs_argmax(logits.data_ptr(), logits.stride(0), n, V, out.data_ptr(), scratch.data_ptr(), _stream()),
           kernels=2 if V >= 16384 else 1)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor, out: torch.Tensor,
           advance: bool = False) -> None:
    """A seeded draw per row from (seed, counter). `advance`: every row's counter goes up by one inside the kernel
    (greedy rows' too), so that a generation loop needs no launch of its own for that."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    n, V = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                        (seeds, "seeds", torch.int64), (counters, "counters", torch.int64)):
        _need(t, name, dt)
        if t.numel() < n:
            raise KernelError(f"{name} has {t.numel()} entries for {n} rows")
    _check(load().xs_sample(logits.data_ptr(), logits.stride(0), n, V, temperature.data_ptr(), top_k.data_ptr(),
                            top_p.data_ptr(), min_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(),
                            1 if advance else 0, out.data_ptr(), _stream()))


def apply_penalties(logits: torch.Tensor, seen: torch.Tensor, gen_count: torch.Tensor, state_rows: torch.Tensor,
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(seen, "seen", torch.uint8); _need(gen_count, "counts", torch.int32)
    n, V = logits.shape
    _check(load().xs_apply_penalties(logits.data_ptr(), logits.stride(0), n, V, seen.data_ptr(), gen_count.data_ptr(),
                                     state_rows.data_ptr(), repetition.data_ptr(), presence.data_ptr(),
                                     frequency.data_ptr(), _stream()))


def note_tokens(tokens: torch.Tensor, rows_of_token: torch.Tensor, seen: torch.Tensor, gen_count: torch.Tensor,
                generated: bool) -> None:
    _need(tokens, "tokens", torch.int32); _need(rows_of_token, "rows", torch.int32)
    V = seen.shape[1]
    _check(load().xs_note_tokens(tokens.data_ptr(), rows_of_token.data_ptr(), tokens.numel(), V, seen.data_ptr(),
                                 gen_count.data_ptr(), 1 if generated else 0, _stream()))
