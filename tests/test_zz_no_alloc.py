"""The allocation-free attention entry point (csrc/xs_no_alloc.h), called through its exported C
symbol exactly as a caller without an allocator would: raw device pointers in, no scratch buffer.
Its result must equal the ordinary entry point's (same kernels, same arithmetic; only where the
partial results are kept differs) on two different problems in a row, and a problem that does not
fit the built-in array must be refused. The file's name makes pytest collect it last."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from xpu_serve_b200.csrc import build
    lib = ctypes.CDLL(build.build(verbose=False))
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    lib.xs_attention_mma_static.argtypes = [P, P, P, I, P, P, P, L, P, I, I, I, I, I, I, I, F, I, I, P]
    lib.xs_attention_mma_static.restype = I
    lib.xs_attention_mma_static_capacity.restype = L
    lib.xs_last_error.restype = ctypes.c_char_p
    return lib


def _problem(seed, kv_lens, Hq, Hkv, D):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = len(kv_lens)
    P = max(-(-L // 64) for L in kv_lens)
    pool = torch.randn(n * P + 1, 2, Hkv, 64, D, generator=g).to(torch.bfloat16).cuda()
    table = torch.randperm(n * P, generator=g).reshape(n, P).to(torch.int32).cuda()
    q = torch.randn(n, Hq, D, generator=g).to(torch.bfloat16).cuda()          # one new token a sequence
    cu = torch.arange(n + 1, dtype=torch.int32).cuda()
    lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    return q, pool, table, cu, lens


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from xpu_serve_b200.ops import lib as ops
    lib = _library()
    assert lib.xs_attention_mma_static_capacity() == 8 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(1, [700, 64, 1, 333], 8, 2, 64, 4), (2, [2000, 1500], 6, 3, 32, 7)]
    for seed, kv_lens, Hq, Hkv, D, splits in cases:
        q, pool, table, cu, lens = _problem(seed, kv_lens, Hq, Hkv, D)
        n = len(kv_lens)
        scale = 1.0 / math.sqrt(D)
        want = torch.empty_like(q)
        scratch = torch.empty(ops.attention_mma_scratch_bytes(n * Hq, D, splits), dtype=torch.uint8, device="cuda")
        ops.attention_mma(q, pool, table, cu, lens, None, want, scratch, n, 1, Hkv, 64, scale, 0, splits)
        got = torch.full_like(q, float("nan"))
        rc = lib.xs_attention_mma_static(q.data_ptr(), pool.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
                                         lens.data_ptr(), None, 0, got.data_ptr(), n, n, 1, Hq, Hkv, D, 64, scale, 0,
                                         splits, stream)
        assert rc == 0, lib.xs_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        gap = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
        assert gap <= 6e-3, f"gap {gap:.3e}"          # the bfloat16 tolerance of the kernel tests; in fact the bits agree
        assert torch.equal(got, want)
    # too large for the built-in array: refused, nothing written
    q, pool, table, cu, lens = _problem(3, [100], 32, 8, 128)
    big_T = 4096
    rc = lib.xs_attention_mma_static(q.data_ptr(), pool.data_ptr(), table.data_ptr(), 2, cu.data_ptr(), lens.data_ptr(),
                                     None, 0, q.data_ptr(), big_T, 1, big_T, 32, 8, 128, 64, 0.1, 0, 8, stream)
    assert rc != 0 and b"built-in array holds" in lib.xs_last_error()
