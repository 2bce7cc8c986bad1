"""The allocation-free attention entry point (csrc/xs_no_alloc.h), called through its exported C
symbol exactly as a caller without an allocator would: raw device pointers in, no scratch buffer.
Its result must equal the ordinary entry point's (same kernels, same arithmetic; only where the
partial results are kept differs) and lie within the kernel tests' tolerance of a float64 reference, on
several different problems in a row (decoding; a window with a gate per head; a few tokens a sequence
right after a larger problem, so that the array still holds partial results of another layout), and a
problem that does not fit the built-in array must be refused. The file's name makes pytest collect it last."""
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


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from test_kernels_gpu import Paged, close
    from xpu_serve_b200.ops import lib as ops
    lib = _library()
    assert lib.xs_attention_mma_static_capacity() == 8 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    cases = [   # starts, q_lens, Hq, Hkv, D, window, gate, splits
        ([699, 63, 0, 332], [1, 1, 1, 1], 8, 2, 64, 0, False, 4),
        ([1999, 1499], [1, 1], 6, 3, 32, 0, False, 7),
        ([700, 130, 260], [1, 1, 1], 8, 2, 64, 50, True, 3),          # a window, a gate per head
        ([3000, 2500, 100], [1, 1, 1], 32, 8, 64, 0, False, 40),      # a large problem: most of the array is written
        ([900, 40], [7, 3], 4, 2, 64, 0, True, 5),                    # then a few tokens a sequence, another layout
    ]
    for seed, (starts, q_lens, Hq, Hkv, D, window, gated, splits) in enumerate(cases):
        pg = Paged(starts, q_lens, Hq, Hkv, D, "bfloat16", seed=seed + 1)
        pg.fill_pool()
        d = pg.dev()
        q, pool, table, cu, lens = d["q"], d["pool"], d["table"], d["cu"], d["kv_lens"]
        n, T = len(starts), sum(q_lens)
        scale = 1.0 / math.sqrt(D)
        gate = torch.randn(T, Hq + 3).to(torch.bfloat16) if gated else None
        gate_dev = None if gate is None else gate.cuda()
        want = torch.empty_like(q)
        scratch = torch.empty(ops.attention_mma_scratch_bytes(T * Hq, D, splits), dtype=torch.uint8, device="cuda")
        ops.attention_mma(q, pool, table, cu, lens, None if gate_dev is None else gate_dev[:, :Hq], want, scratch, n,
                          max(q_lens), Hkv, 64, scale, window, splits)
        got = torch.full_like(q, float("nan"))
        rc = lib.xs_attention_mma_static(q.data_ptr(), pool.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
                                         lens.data_ptr(), None if gate_dev is None else gate_dev.data_ptr(),
                                         0 if gate_dev is None else gate_dev.stride(0), got.data_ptr(), T, n, max(q_lens),
                                         Hq, Hkv, D, 64, scale, window, splits, stream)
        assert rc == 0, lib.xs_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        close(got, pg.reference(scale, window, None if gate is None else gate[:, :Hq]), "bfloat16", factor=3)
        assert torch.equal(got, want), "the two entry points run the same kernels: their bits agree"
    # too large for the built-in array: refused, nothing written
    q = torch.zeros(1, 32, 128, dtype=torch.bfloat16, device="cuda")
    pool = torch.zeros(3, 2, 8, 64, 128, dtype=torch.bfloat16, device="cuda")
    table = torch.zeros(1, 2, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    lens = torch.tensor([100], dtype=torch.int32, device="cuda")
    big_T = 4096
    rc = lib.xs_attention_mma_static(q.data_ptr(), pool.data_ptr(), table.data_ptr(), 2, cu.data_ptr(), lens.data_ptr(),
                                     None, 0, q.data_ptr(), big_T, 1, big_T, 32, 8, 128, 64, 0.1, 0, 8, stream)
    assert rc != 0 and b"built-in array holds" in lib.xs_last_error()
