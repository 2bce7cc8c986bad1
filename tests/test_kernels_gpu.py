"""Each CUDA kernel alone against a plain PyTorch float64 reference of the same operation, at
sizes other than the tiny models': widths and vocabularies that are no power of two, head sizes
in steps of 16, several head-group ratios, ragged batches, shuffled page tables. Where random
inputs would hide a fault (a far key, a window's edge), one query and key are scaled so that a
single score dominates."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# largest |difference| / largest |reference|: float32 sums of <= 4096 products; bfloat16 outputs are
# rounded to 8 bits (2^-9 relative) on top of bfloat16 inputs that both sides share
TOL = {"float32": 2e-6, "bfloat16": 6e-3}


def ops():
    from xpu_serve_b200.ops import lib
    return lib


def close(got, ref, dtype, factor=1.0):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all()
    gap = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert gap <= TOL[dtype] * factor, f"gap {gap:.3e}"


def gap_ok(got, ref, rel=2e-2):
    got, ref = got.double().cpu(), ref.double().cpu()
    return (got - ref).abs().max().item() <= rel * ref.abs().max().item()


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------ embedding, norms, activation
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    V, H = 1003, 200
    table = torch.randn(V, H, device=DEV).to(DT[dtype])
    ids = torch.tensor([0, 1002, 17, 17, 500], dtype=torch.int32, device=DEV)
    h = torch.empty(5, H, device=DEV)
    ops().embed(table, ids, h)
    assert torch.equal(h, table[ids.long()].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [96, 200, 2048, 5000])
def test_add_rmsnorm_all_forms(dtype, H):
    T, eps, eps_post = 7, 1e-5, 3e-6
    h0 = torch.randn(T, H, device=DEV) * 3
    m = torch.randn(T, H, device=DEV).to(DT[dtype])
    w = torch.rand(H, device=DEV) + 0.5
    pw = torch.rand(H, device=DEV) + 0.5
    # plain norm
    y = torch.empty(T, H, device=DEV, dtype=DT[dtype])
    h = h0.clone()
    ops().add_rmsnorm(h, None, None, w, y, None, eps)
    close(y, rms_norm(h0.double(), w.double(), eps), dtype)
    assert torch.equal(h, h0)
    # add then norm
    h = h0.clone()
    ops().add_rmsnorm(h, m, None, w, y, None, eps)
    s = h0.double() + m.double()
    close(h, s, "float32")
    close(y, rms_norm(s, w.double(), eps), dtype)
    # sandwich: the branch is normed (with its own eps) before it joins the stream
    h = h0.clone()
    ops().add_rmsnorm(h, m, pw, w, y, None, eps, eps_post)
    s = h0.double() + rms_norm(m.double(), pw.double(), eps_post)
    close(h, s, "float32")
    close(y, rms_norm(s, w.double(), eps), dtype)
    # chosen rows only, packed
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    h = h0.clone()
    y3 = torch.empty(3, H, device=DEV, dtype=DT[dtype])
    ops().add_rmsnorm(h, m, None, w, y3, rows, eps)
    close(y3, rms_norm((h0.double() + m.double())[rows.long()], w.double(), eps), dtype)
    # flush without a norm
    h = h0.clone()
    ops().add_rmsnorm(h, m, pw, None, None, None, eps, eps_post)
    close(h, h0.double() + rms_norm(m.double(), pw.double(), eps_post), "float32")


def test_add_rmsnorm_uses_each_eps_where_it_belongs():
    """A small branch makes its norm's eps matter; swapping the two eps must show."""
    T, H, eps, eps_post = 4, 80, 1e-5, 3e-6
    h0 = torch.randn(T, H, device=DEV)
    m = torch.randn(T, H, device=DEV) * 2e-3
    w, pw = torch.rand(H, device=DEV) + 0.5, torch.rand(H, device=DEV) + 0.5
    y = torch.empty(T, H, device=DEV)
    h = h0.clone()
    ops().add_rmsnorm(h, m, pw, w, y, None, eps, eps_post)
    right = h0.double() + rms_norm(m.double(), pw.double(), eps_post)
    swapped = h0.double() + rms_norm(m.double(), pw.double(), eps)
    close(h, right, "float32")
    assert (h.double() - swapped).abs().max() > 1e-2


def test_rmsnorm_has_no_plus_one_offset():
    H = 64
    h = torch.randn(3, H, device=DEV)
    w = torch.rand(H, device=DEV)
    y = torch.empty(3, H, device=DEV)
    ops().add_rmsnorm(h, None, None, w, y, None, 1e-5)
    wrong = rms_norm(h.double(), 1.0 + w.double(), 1e-5)
    assert (y.double() - wrong).abs().max() > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(dtype):
    T, F = 5, 333
    gu = (torch.randn(T, 2 * F + 6, device=DEV) * 3).to(DT[dtype])     # a padded row stride
    out = torch.empty(T, F, device=DEV, dtype=DT[dtype])
    ops().silu_mul(gu[:, :2 * F], out)
    g, u = gu[:, :F].double(), gu[:, F:2 * F].double()
    close(out, g / (1 + torch.exp(-g)) * u, dtype)


def test_silu_mul_interleaved_blocks_of_eight():
    T, F = 9, 336
    g = torch.randn(T, F, device=DEV) * 3
    u = torch.randn(T, F, device=DEV)
    gu = torch.stack([g.view(T, F // 8, 8), u.view(T, F // 8, 8)], 2).reshape(T, 2 * F)
    want = g.double() / (1 + torch.exp(-g.double())) * u.double()
    for dtype in ("float32", "bfloat16"):
        x = gu.to(DT[dtype])
        out = torch.empty(T, F, device=DEV, dtype=DT[dtype])
        ops().silu_mul(x, out, interleave=8)
        gg, uu = x.view(T, F // 8, 2, 8)[:, :, 0].reshape(T, F).double(), x.view(T, F // 8, 2, 8)[:, :, 1].reshape(T, F).double()
        close(out, gg / (1 + torch.exp(-gg)) * uu, dtype)
        assert gap_ok(out, want)            # and the layout is the intended one: close to the unrounded values too


# ---------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 100, 96), (65, 130, 200), (200, 1000, 333), (9, 64, 4096)])
def test_gemm_generic(dtype, M, N, K):
    x = torch.randn(M, K, device=DEV).to(DT[dtype])
    w = torch.randn(N, K, device=DEV).to(DT[dtype])
    bias = torch.randn(N, device=DEV)
    out = torch.empty(M, N, device=DEV)
    ops().gemm_generic(x, w, out, bias)
    close(out, x.double() @ w.double().T + bias.double(), "float32", factor=math.sqrt(K) / 8 + 1)
    wrong = x.double() @ w.double().flip(0).T + bias.double()
    assert (out.double() - wrong).abs().max() > 0.1 or N == 1
    if dtype == "bfloat16":
        o2 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        ops().gemm_generic(x, w, o2)
        close(o2, x.double() @ w.double().T, "bfloat16")


def test_gemm_generic_rows_do_not_depend_on_the_batch():
    K, N = 777, 150
    x = torch.randn(40, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    full = torch.empty(40, N, device=DEV)
    one = torch.empty(1, N, device=DEV)
    ops().gemm_generic(x, w, full)
    ops().gemm_generic(x[17:18], w, one)
    assert torch.equal(full[17:18], one)


@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 16])
# the two widest: more row tiles than CTAs fit on the device at once; (2048, 8192), (4096, 1024): no edge anywhere;
# (2048, 8192), (3072, 2048), (512, 4096): few row tiles and K a multiple of 2,048, the variant of sixteen loads a round
# (256, 1536), (2048, 10752), (48, 192), (64, 64): no edge but K is no multiple of 1,024: a short last round
@pytest.mark.parametrize("N,K", [(16, 32), (100, 96), (1000, 200), (2048, 8192), (333, 2056), (10007, 200), (20000, 1096), (4096, 1024),
                                 (3072, 2048), (512, 4096), (256, 1536), (2048, 10752), (48, 192), (64, 64)])
def test_gemm_small_m(M, N, K):
    lib = ops()
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    assert lib.gemm_small_m_supports(M, K, x.stride(0), w.stride(0))
    ref = x.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    lib.gemm_small_m(x, w, out)
    close(out, ref, "float32", factor=4)
    out16 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    lib.gemm_small_m(x, w, out16, bias)
    close(out16, ref + bias.double(), "bfloat16")
    res = torch.randn(M, N, device=DEV)
    want = res.double() + ref
    lib.gemm_small_m(x, w, None, None, residual=res)
    close(res, want, "float32", factor=4)
    one = torch.empty(1, N, device=DEV)
    lib.gemm_small_m(x[M - 1:M], w, one)
    assert torch.equal(one, out[M - 1:M]), "a row's result depends on the batch"


@pytest.mark.parametrize("M,N,K,ksplit", [(8, 2048, 8192, 4), (3, 100, 4104, 3), (16, 256, 2048, 8), (1, 48, 512, 2), (5, 2048, 2048, 7),
                                          (8, 2048, 8192, 2), (6, 1024, 6144, 3), (8, 2048, 10752, 4), (4, 512, 6656, 2),
                                          (16, 256, 1536, 3)])
def test_gemm_small_m_k_slices(M, N, K, ksplit):
    """K cut into slices over several CTAs: the last CTA of a tile to arrive adds the slices in slice order, so
    the bits do not depend on which one that was; a second and third call find the counters reset."""
    lib = ops()
    g = torch.Generator(device="cpu").manual_seed(N + ksplit)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    ref = x.double() @ w.double().T + bias.double()
    scratch = torch.zeros(lib.gemm_small_m_scratch_bytes(M, N, ksplit), dtype=torch.uint8, device=DEV)
    outs = []
    for _ in range(3):
        out = torch.full((M, N), float("nan"), device=DEV)
        lib.gemm_small_m(x, w, out, bias, ksplit=ksplit, scratch=scratch)
        close(out, ref, "float32", factor=4)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    res = torch.randn(M, N, generator=g).to(DEV)
    want = res.double() + ref
    lib.gemm_small_m(x, w, None, bias, residual=res, ksplit=ksplit, scratch=scratch)
    close(res, want, "float32", factor=4)


@pytest.mark.parametrize("M,H,K,taps,bias", [(8, 2048, 2048, 3, False), (1, 64, 64, 7, True), (5, 96, 200, 2, False), (13, 160, 72, 8, True),
                                             (8, 1024, 512, 4, False)])
def test_gemm_small_m_with_the_convolution_behind_it(M, H, K, taps, bias):
    """in_proj and, in the tail of the same kernel, the gated convolution of one token a sequence with its state's
    update: against a float64 restatement, bit for bit against the convolution kernel of its own, three steps in
    a row (the counters must come back to zero), shuffled slots, neighbouring slots untouched."""
    lib = ops()
    g = torch.Generator(device="cpu").manual_seed(M * H + taps)
    w = (torch.randn(3 * H, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    b_in = torch.randn(3 * H, generator=g).to(DEV) if bias else None
    w_t = torch.randn(taps, H, generator=g).to(DEV)
    b_conv = torch.randn(H, generator=g).to(DEV) if bias else None
    n_slots = M + 3
    slots = torch.randperm(n_slots, generator=g)[:M].to(torch.int32).to(DEV)
    state0 = torch.randn(n_slots, taps - 1, H, generator=g).to(torch.bfloat16).to(DEV)
    fused_state, split_state = state0.clone(), state0.clone()
    ref_state = state0.double().cpu()
    counters = torch.zeros(max(H // 16, 1), dtype=torch.int32, device=DEV)
    seq_of = torch.arange(M, dtype=torch.int32, device=DEV)
    cu = torch.arange(M + 1, dtype=torch.int32, device=DEV)
    for step in range(3):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        bcx = torch.full((M, 3 * H), float("nan"), device=DEV, dtype=torch.bfloat16)
        y = torch.full((M, H), float("nan"), device=DEV, dtype=torch.bfloat16)
        lib.gemm_small_m(x, w, bcx, b_in, conv=dict(taps=w_t, bias=b_conv, state=fused_state, slots=slots, out=y, counters=counters))
        assert int(counters.abs().sum()) == 0, "the counters were not left at zero"
        # the same in two kernels
        bcx2 = torch.empty_like(bcx)
        lib.gemm_small_m(x, w, bcx2, b_in)
        assert torch.equal(bcx, bcx2)
        y2 = torch.empty_like(y)
        lib.short_conv(bcx2, w_t, b_conv, split_state, seq_of, cu, slots, y2, all_single=True)
        assert torch.equal(y, y2) and torch.equal(fused_state, split_state), "the fused tail and the kernel of its own differ"
        # float64, from the bfloat16 values of B, C, X that both read
        b, c, xx = bcx.double().cpu()[:, :H], bcx.double().cpu()[:, H:2 * H], bcx.double().cpu()[:, 2 * H:]
        gg = (b * xx).to(torch.bfloat16).double()
        sl = slots.cpu().long()
        acc = (b_conv.double().cpu() if bias else 0) + (w_t.double().cpu()[:-1, None, :] * ref_state[sl].transpose(0, 1)).sum(0) \
            + w_t.double().cpu()[-1] * gg
        close(y, acc * c, "bfloat16", factor=2)
        ref_state[sl] = torch.cat([ref_state[sl][:, 1:], gg[:, None, :]], 1)
        assert torch.equal(fused_state.double().cpu(), ref_state), "the state holds other values than the inputs that went by"


@pytest.mark.parametrize("M,N,K,ksplit", [(8, 65536, 256, 1), (1, 1000, 96, 1), (5, 20011, 64, 1), (16, 512, 4096, 2), (3, 48, 32, 1)])
def test_gemm_small_m_with_the_argmax_behind_it(M, N, K, ksplit):
    """The head product leaves every row's most likely column beside the logits: the lowest column among equal
    values (planted: equal rows of the weight far apart, in other CTAs' tiles), rows of negative values only, three
    calls in a row (keys and counter must come back to zero)."""
    lib = ops()
    g = torch.Generator(device="cpu").manual_seed(N + M)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    w[N - 2] = w[7]                                        # equal logits in tiles far apart: the lower column wins
    w[N // 2] = w[7]
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    x[0] = (w[7].float() * 4).to(torch.bfloat16)           # row 0 points at column 7 (and its copies)
    w, x = w.to(DEV), x.to(DEV)
    bias = torch.randn(N, generator=g).to(DEV) * 0.01
    bias[N - 2] = bias[N // 2] = bias[7]
    keys = torch.zeros(16, dtype=torch.int64, device=DEV)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    scratch = torch.zeros(lib.gemm_small_m_scratch_bytes(M, N, ksplit), dtype=torch.uint8, device=DEV) if ksplit > 1 else None
    for call in range(3):
        shift = 0.0 if call < 2 else -50.0                 # the last call: every logit negative
        out = torch.empty(M, N, device=DEV)
        best = torch.full((M,), -7, dtype=torch.int32, device=DEV)
        lib.gemm_small_m(x, w, out, bias + shift, ksplit=ksplit, scratch=scratch, argmax=(best, keys, counter))
        assert int(keys.abs().sum()) == 0 and int(counter.item()) == 0
        want = torch.empty(M, dtype=torch.int32, device=DEV)
        lib.argmax(out, want)
        assert torch.equal(best, want), (best.tolist(), want.tolist())
        assert (out.argmax(1) == best).all() or out[0, 7] == out[0, N // 2]
        assert best[0].item() == 7
        if call == 2:
            assert (out.max(1).values < 0).all()


@pytest.mark.parametrize("F", [344, 10400])
@pytest.mark.parametrize("M", [1, 7, 8, 13])
def test_gemm_small_m_with_fused_activation(M, F):
    lib = ops()
    K = 200
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    gate = (torch.randn(F, K, device=DEV) / math.sqrt(K) * 3).to(torch.bfloat16)
    up = (torch.randn(F, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    w = torch.stack([gate.view(F // 8, 8, K), up.view(F // 8, 8, K)], 1).reshape(2 * F, K).contiguous()
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    out = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    lib.gemm_small_m(x, w, out, swiglu=True)
    close(out, g / (1 + torch.exp(-g)) * u, "bfloat16")


@pytest.mark.parametrize("M,H,N2,K1,ks1,ks2", [(8, 2048, 512, 1024, 2, 1), (3, 200, 96, 64, 1, 1), (13, 2304, 256, 512, 4, 2),
                                                (1, 64, 48, 4096, 4, 1), (8, 2048, 16384, 1024, 2, 1), (5, 96, 9616, 64, 1, 1),
                                                (8, 2048, 512, 4096, 2, 1)])
def test_gemm_small_m_carries_the_norm(M, H, N2, K1, ks1, ks2):
    """Two products with an RMSNorm between them and no norm kernel: the first adds to the float32 stream and
    leaves stream * weight and per-tile sums of squares, the second scales its rows by 1 / rms. Widths that
    are no multiple of 16, more tiles than the kernel stages in shared memory (2304 / 16 = 144), K slices on
    either side, and a row whose stream is a thousand times larger than its neighbours'."""
    lib = ops()
    g = torch.Generator(device="cpu").manual_seed(M * H)
    act = torch.randn(M, K1, generator=g).to(torch.bfloat16).to(DEV)
    w1 = (torch.randn(H, K1, generator=g) / math.sqrt(K1)).to(torch.bfloat16).to(DEV)
    h0 = torch.randn(M, H, generator=g).to(DEV)
    h0[M // 2] *= 1000.0
    nw = (torch.rand(H, generator=g) + 0.5).to(DEV)
    bias1 = torch.randn(H, generator=g).to(DEV)
    w2 = (torch.randn(N2, H, generator=g) / math.sqrt(H)).to(torch.bfloat16).to(DEV)
    bias2 = torch.randn(N2, generator=g).to(DEV)
    eps = 1e-5
    scratch = torch.zeros(8 << 20, dtype=torch.uint8, device=DEV)
    h = h0.clone()
    nx = torch.full((M, H), float("nan"), device=DEV, dtype=torch.bfloat16)
    ssq = torch.full(((H + 15) // 16, 16), float("nan"), device=DEV)
    lib.gemm_small_m(act, w1, None, bias1, residual=h, ksplit=ks1, scratch=scratch if ks1 > 1 else None,
                     next_w=nw, next_x=nx, out_ssq=ssq)
    h_ref = h0.double() + act.double() @ w1.double().T + bias1.double()
    close(h, h_ref, "float32", factor=4)
    close(nx, h_ref * nw.double(), "bfloat16")
    close(ssq[:, :M].sum(0), (h_ref ** 2).sum(1), "float32", factor=4)
    normed = h_ref / torch.sqrt((h_ref ** 2).mean(1, keepdim=True) + eps) * nw.double()
    ref = normed @ w2.double().T + bias2.double()
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N2), float("nan"), device=DEV, dtype=out_dtype)
        lib.gemm_small_m(nx, w2, out, bias2, ksplit=ks2, scratch=scratch if ks2 > 1 else None, in_ssq=ssq, in_width=H,
                         in_eps=eps)
        close(out, ref, "bfloat16", factor=2)
    if N2 % 16 == 0:       # the same through the fused activation: w2's rows as 8 gates, 8 ups
        F = N2 // 2
        o = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
        lib.gemm_small_m(nx, w2, o, swiglu=True, in_ssq=ssq, in_width=H, in_eps=eps)
        pre = (normed @ w2.double().T).view(M, F // 8, 2, 8)
        gate, up = pre[:, :, 0].reshape(M, F), pre[:, :, 1].reshape(M, F)
        close(o, gate / (1 + torch.exp(-gate)) * up, "bfloat16", factor=2)


TC_SHAPES = [(1, 128, 64), (8, 256, 128), (16, 2048, 2048), (5, 100, 96), (33, 1000, 200), (64, 384, 512),
             (130, 300, 264), (700, 1024, 2048), (2048, 512, 1024), (100, 300, 256), (128, 128, 64),
             (257, 2048, 2048), (1000, 6144, 512)]


@pytest.mark.parametrize("T,N,K", TC_SHAPES)
def test_gemm_tc_store_and_residual(T, N, K):
    lib = ops()
    g = torch.Generator(device="cpu").manual_seed(T + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    assert lib.gemm_tc_supports(T, N, K, x.stride(0), w.stride(0))
    ref = x.double() @ w.double().T
    status = lib.gemm_tc_status(DEV)
    out = torch.full((T, N), float("nan"), device=DEV)
    lib.gemm_tc(x, w, out)
    torch.cuda.synchronize()
    assert status.item() == 0, "a wait inside the kernel gave up"
    close(out, ref, "float32", factor=4)
    out16 = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    lib.gemm_tc(x, w, out16, bias)
    close(out16, ref + bias.double(), "bfloat16")
    res = torch.randn(T, N, device=DEV)
    want = res.double() + ref
    lib.gemm_tc(x, w, res, epilogue=lib.EPI_RESIDUAL)
    close(res, want, "float32", factor=4)
    if T > 1:
        one = torch.empty(1, N, device=DEV)
        lib.gemm_tc(x[T - 1:T], w, one)
        close(one, ref[T - 1:T], "float32", factor=4)
    assert status.item() == 0


@pytest.mark.parametrize("T,F,K,ksplit", [(1, 344, 200, 1), (8, 1024, 2048, 1), (16, 256, 4096, 4), (40, 136, 512, 2), (300, 512, 256, 1)])
def test_gemm_tc_swiglu_and_k_slices(T, F, K, ksplit):
    lib = ops()
    g = torch.Generator(device="cpu").manual_seed(F)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(F, K, generator=g) / math.sqrt(K) * 3).to(torch.bfloat16).to(DEV)
    up = (torch.randn(F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    w = torch.stack([gate.view(F // 8, 8, K), up.view(F // 8, 8, K)], 1).reshape(2 * F, K).contiguous()
    gg, uu = x.double() @ gate.double().T, x.double() @ up.double().T
    scratch = torch.zeros(max(lib.gemm_tc_scratch_bytes(T, 2 * F, ksplit), 16), dtype=torch.uint8, device=DEV)
    out = torch.empty(T, F, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):          # the counters must be left ready for the next call
        out.fill_(float("nan"))
        lib.gemm_tc(x, w, out, epilogue=lib.EPI_SWIGLU, ksplit=ksplit, scratch=scratch if ksplit > 1 else None)
        close(out, gg / (1 + torch.exp(-gg)) * uu, "bfloat16")
    plain_out = torch.empty(T, 2 * F, device=DEV)
    lib.gemm_tc(x, w, plain_out, ksplit=ksplit, scratch=scratch if ksplit > 1 else None)
    close(plain_out, x.double() @ w.double().T, "float32", factor=4)
    assert lib.gemm_tc_status(DEV).item() == 0


def test_gemm_small_m_refuses_what_it_cannot_take():
    lib = ops()
    assert not lib.gemm_small_m_supports(17, 64, 64, 64)
    assert not lib.gemm_small_m_supports(4, 100, 100, 100)      # K is no multiple of 8
    x = torch.zeros(4, 100, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(8, 100, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(lib.KernelError, match="not supported"):
        lib.gemm_small_m(x, w, torch.empty(4, 8, device=DEV))


# -------------------------------------------------------------------------------- attention
class Paged:
    """A ragged batch with a shuffled page table, and dense float64 copies for the reference."""

    def __init__(self, starts, q_lens, Hq, Hkv, D, dtype, seed=0, page=64):
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.starts, self.q_lens, self.Hq, self.Hkv, self.D, self.page = starts, q_lens, Hq, Hkv, D, page
        n = len(starts)
        self.kv_lens = [s + q for s, q in zip(starts, q_lens)]
        P = max(-(-L // page) for L in self.kv_lens)
        n_pages = n * P + 3
        perm = torch.randperm(n_pages, generator=g)
        self.table = perm[:n * P].reshape(n, P).to(torch.int32)
        self.pool = (torch.randn(n_pages, 2, Hkv, page, D, generator=g) * 50).to(DT[dtype])   # stale contents are loud
        self.k = [torch.randn(L, Hkv, D, generator=g) for L in self.kv_lens]
        self.v = [torch.randn(L, Hkv, D, generator=g) for L in self.kv_lens]
        T = sum(q_lens)
        self.q = torch.randn(T, Hq, D, generator=g)
        self.cu = np.concatenate([[0], np.cumsum(q_lens)])
        self.seq_of = np.repeat(np.arange(n), q_lens)
        self.pos = np.concatenate([np.arange(s, s + q) for s, q in zip(starts, q_lens)])

    def fill_pool(self, upto_start_only=False):
        for s in range(len(self.starts)):
            L = self.starts[s] if upto_start_only else self.kv_lens[s]
            for j in range(L):
                pg, r = int(self.table[s, j // self.page]), j % self.page
                self.pool[pg, 0, :, r] = self.k[s][j].to(self.pool.dtype)
                self.pool[pg, 1, :, r] = self.v[s][j].to(self.pool.dtype)

    def drop_pages_behind(self, window):
        """What the cache does behind a window: pages that no query of this step can see are given back and the
        table says -1 there (their storage now belongs to somebody else: it is made loud)."""
        dropped = 0
        for s, start in enumerate(self.starts):
            first = max(0, start - window + 1) // self.page
            for lp in range(first):
                self.pool[int(self.table[s, lp])] = 1e4
                self.table[s, lp] = -1
                dropped += 1
        return dropped

    def dev(self):
        i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)   # noqa: E731
        return dict(pool=self.pool.to(DEV), table=self.table.to(DEV), cu=i32(self.cu), seq_of=i32(self.seq_of),
                    pos=i32(self.pos), kv_lens=i32(self.kv_lens), q=self.q.to(DEV).to(self.pool.dtype))

    def reference(self, scale, window, gate=None):
        q = self.q.to(self.pool.dtype).double()
        out = torch.zeros_like(q)
        G = self.Hq // self.Hkv
        for t in range(q.shape[0]):
            s, p = int(self.seq_of[t]), int(self.pos[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            k = self.k[s].to(self.pool.dtype).double()[lo:p + 1]
            v = self.v[s].to(self.pool.dtype).double()[lo:p + 1]
            for h in range(self.Hq):
                sc = scale * (k[:, h // G] @ q[t, h])
                pr = torch.softmax(sc, 0)
                out[t, h] = pr @ v[:, h // G]
                if gate is not None:
                    out[t, h] *= torch.sigmoid(gate[t, h].double())
        return out


ATTN_CASES = [
    # starts, q_lens, Hq, Hkv, D, window
    ([0], [1], 4, 2, 16, 0),
    ([0, 0, 0], [5, 70, 129], 4, 2, 32, 0),          # prompts of unequal lengths
    ([63, 64, 200, 0], [1, 1, 1, 1], 8, 1, 64, 0),   # decode; one sequence holds a single key
    ([10, 100], [60, 3], 6, 3, 48, 0),               # continuing sequences with several new tokens
    ([0, 130], [150, 1], 4, 1, 32, 37),              # a window with its edge inside and across pages
    ([300], [1], 3, 1, 96, 64),
    ([0], [200], 32, 8, 64, 0),                      # the 1.2B shape's heads
    ([500, 37, 1999], [1, 1, 1], 16, 2, 128, 0),
    ([0], [90], 5, 5, 80, 17),                       # a head size only the generic kernel takes
    ([4100, 30], [1, 1], 8, 2, 64, 0),               # more than 32 blocks of keys: 40 splits all hold some
    ([500], [200], 16, 1, 64, 100),                  # a piece of a prompt behind a window that has left pages behind
    ([700, 130, 260], [1, 1, 1], 8, 2, 64, 50),      # decoding behind such a window
]


@pytest.mark.parametrize("case", ATTN_CASES)
@pytest.mark.parametrize("kernel,dtype", [("generic", "float32"), ("generic", "bfloat16"), ("mma", "bfloat16")])
def test_attention(case, kernel, dtype):
    lib = ops()
    starts, q_lens, Hq, Hkv, D, window = case
    if kernel == "mma" and not lib.attention_mma_supports(D, 64, Hq // Hkv):
        with pytest.raises(lib.KernelError, match="not supported"):
            run_attention(lib, Paged([0], [1], Hq, Hkv, D, dtype), kernel, 0.1, 0, None, 1)
        return
    pg = Paged(starts, q_lens, Hq, Hkv, D, dtype, seed=len(starts) + D)
    # plant one dominant score: the first visible key of the last query of every sequence
    for s in range(len(starts)):
        t = int(pg.cu[s + 1]) - 1
        p = int(pg.pos[t])
        j = max(0, p - window + 1) if window > 0 else 0
        pg.k[s][j] = pg.q[t, 0] * 3.0
        if window > 0 and j > 0:
            pg.k[s][j - 1] = pg.q[t, 0] * 6.0          # just outside the window: must not be seen
    pg.fill_pool()
    scale = 1.0 / math.sqrt(D)
    gate = torch.randn(sum(q_lens), Hq + 3).to(DT[dtype])
    for trimmed in ((False, True) if window > 0 else (False,)):
        if trimmed and pg.drop_pages_behind(window) == 0:
            continue
        for gt in (None, gate):
            ref = pg.reference(scale, window, None if gt is None else gt[:, :Hq])
            for splits in ([1] if kernel == "generic" else [1, 2, 5, 40]):
                out = run_attention(lib, pg, kernel, scale, window, gt, splits)
                close(out, ref, dtype, factor=3 if dtype == "bfloat16" else 20)
                if kernel == "mma" and splits > 1 and max(q_lens) == 1:
                    # one token a sequence: the key splits merged by the last CTA to finish, bit for bit the combine
                    # kernel's result, the counters back at zero, twice in a row
                    counters = torch.zeros(len(starts) * Hkv, dtype=torch.int32, device=DEV)
                    for _ in range(2):
                        merged = run_attention(lib, pg, kernel, scale, window, gt, splits, counters=counters)
                        assert torch.equal(merged, out) and int(counters.abs().sum()) == 0
                if kernel == "mma" and max(q_lens) == 1 and D == 64:
                    # head size 64, one token a sequence: the kernel that the TMA unit feeds (pages as whole boxes, swizzled
                    # shared memory, stale rows past a sequence's end and pages given back left as they are and masked)
                    counters = torch.zeros(len(starts) * Hkv, dtype=torch.int32, device=DEV)
                    for with_counters in (False, True):
                        fed = run_attention(lib, pg, kernel, scale, window, gt, splits, tma=True,
                                            counters=counters if with_counters else None)
                        close(fed, ref, dtype, factor=3)
                        assert lib.gemm_tc_status(DEV).item() == 0, "a wait inside the kernel gave up"
                        assert int(counters.abs().sum()) == 0


def test_attention_refuses_more_splits_than_it_combines():
    lib = ops()
    with pytest.raises(lib.KernelError, match="1 to 64 key splits"):
        run_attention(lib, Paged([100], [1], 4, 2, 64, "bfloat16"), "mma", 0.1, 0, None, 65)


ATTN_TC_CASES = [
    # starts, q_lens, Hq, Hkv, window (head size 64)
    ([0], [200], 32, 8, 0),                          # the 1.2B shape's heads: 32 tokens a tile
    ([63, 64, 200, 0], [1, 1, 1, 1], 8, 1, 0),       # single tokens; a sequence that holds one key; a page's first row
    ([0, 0, 0], [5, 70, 300], 4, 2, 0),              # prompts of unequal lengths, several tiles and blocks
    ([10, 100, 700], [60, 3, 130], 4, 4, 0),         # continuing sequences, one head a group
    ([0, 130], [150, 1], 4, 1, 37),                  # a window with its edge inside and across pages
    ([500], [200], 16, 1, 100),                      # 16 heads a group, a window that has left whole blocks behind
    ([300, 0, 129], [40, 7, 2], 4, 2, 50),           # short pieces behind a window, pages given back
    ([0], [129], 2, 2, 0),                           # one row into the second tile, one key into the second block
]


@pytest.mark.parametrize("case", ATTN_TC_CASES)
def test_attention_tc(case):
    """The tcgen05 kernel for prompts against the float64 reference, with a dominant score planted at the first
    visible key of each sequence's last query (a far key; with a window: its very edge) and a larger one just
    outside the window. The cache holds loud stale values wherever the sequences do not."""
    lib = ops()
    starts, q_lens, Hq, Hkv, window = case
    D = 64
    assert lib.attention_tc_supports(D, 64, Hq // Hkv)
    assert not lib.attention_tc_supports(128, 64, 4) and not lib.attention_tc_supports(64, 64, 3)
    pg = Paged(starts, q_lens, Hq, Hkv, D, "bfloat16", seed=len(starts) + Hq)
    for s in range(len(starts)):
        t = int(pg.cu[s + 1]) - 1
        p = int(pg.pos[t])
        j = max(0, p - window + 1) if window > 0 else 0
        pg.k[s][j] = pg.q[t, 0] * 3.0
        if window > 0 and j > 0:
            pg.k[s][j - 1] = pg.q[t, 0] * 6.0
    pg.fill_pool()
    scale = 1.0 / math.sqrt(D)
    gate = torch.randn(sum(q_lens), Hq + 3).to(torch.bfloat16)
    for trimmed in ((False, True) if window > 0 else (False,)):
        # the second time with the pages behind the window given back: -1 in the table, loud values in their storage
        if trimmed and pg.drop_pages_behind(window) == 0:
            continue
        for gt in (None, gate):
            ref = pg.reference(scale, window, None if gt is None else gt[:, :Hq])
            out = run_attention(lib, pg, "tc", scale, window, gt, 1)
            close(out, ref, "bfloat16", factor=3)
            same = run_attention(lib, pg, "mma", scale, window, gt, 1)
            close(out, same.double(), "bfloat16", factor=3)
            # the order in which the CTAs start changes no bit
            assert torch.equal(out, run_attention(lib, pg, "tc_head_after_head", scale, window, gt, 1))


def run_attention(lib, pg, kernel, scale, window, gate, splits, counters=None, tma=False):
    d = pg.dev()
    T = d["q"].shape[0]
    out = torch.full((T, pg.Hq, pg.D), float("nan"), device=DEV, dtype=d["q"].dtype)
    gt = None if gate is None else gate.to(DEV)[:, :pg.Hq]
    if kernel in ("tc", "tc_head_after_head"):
        # (a length beyond what L2 holds for all heads makes the kernel start its CTAs one kv head after the other)
        lib.attention_tc(d["q"], d["pool"], d["table"], d["cu"], d["kv_lens"], gt, out, len(pg.starts), max(pg.q_lens),
                         pg.Hkv, 64, scale, window, max_kv_len=0 if kernel == "tc" else 1 << 24)
        assert lib.gemm_tc_status(DEV).item() == 0, "a wait inside the kernel gave up"
    elif kernel == "generic":
        lib.attention_generic(d["q"], d["pool"], d["table"], d["seq_of"], d["pos"], gt, out, pg.Hkv, 64, scale, window)
    else:
        need = lib.attention_mma_scratch_bytes(T * pg.Hq, pg.D, splits)
        scratch = torch.full((max(need, 1),), 255, dtype=torch.uint8, device=DEV) if splits > 1 else None
        lib.attention_mma(d["q"], d["pool"], d["table"], d["cu"], d["kv_lens"], gt, out, scratch, len(pg.starts),
                          max(pg.q_lens), pg.Hkv, 64, scale, window, splits, counters=counters, bounded_waits=tma)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,pairs,Hq,Hkv", [(16, 8, 4, 2), (32, 16, 3, 1), (48, 12, 6, 3), (64, 32, 8, 8), (128, 20, 2, 1), (256, 128, 2, 1)])
def test_qk_norm_rope_store(dtype, D, pairs, Hq, Hkv):
    lib = ops()
    pg = Paged([0, 70, 5], [9, 1, 66], Hq, Hkv, D, dtype)
    pg.fill_pool(upto_start_only=True)
    d = pg.dev()
    T = sum(pg.q_lens)
    width = (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, width + 8, device=DEV).to(DT[dtype])
    qw, kw = torch.rand(D, device=DEV) + 0.5, torch.rand(D, device=DEV) + 0.5
    eps, theta = 1e-6, 10000.0
    inv = torch.zeros(D // 2, dtype=torch.float64)
    inv[:pairs] = (1.0 / theta ** (2.0 * torch.arange(pairs, dtype=torch.float64) / D)).float().double()
    ang = torch.arange(256, dtype=torch.float64)[:, None] * inv[None, :]
    rope = torch.stack([ang.cos(), ang.sin()], -1).float().to(DEV)
    q_out = torch.empty(T, Hq, D, device=DEV, dtype=DT[dtype])
    before = d["pool"].clone()
    lib.qk_norm_rope_store(qkv, q_out, d["pool"], d["table"], d["seq_of"], d["pos"], qw, kw, rope, Hq, Hkv, D, 64,
                           eps, True)
    x = qkv.double().cpu()
    pos = torch.tensor(pg.pos)

    def norm_rope(v, w):     # v [T, heads, D]
        v = rms_norm(v, w.double().cpu(), eps)
        c, s = ang[pos].cos()[:, None, :], ang[pos].sin()[:, None, :]
        a, b = v[..., :D // 2], v[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    q_ref = norm_rope(x[:, :Hq * D].reshape(T, Hq, D), qw)
    k_ref = norm_rope(x[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D), kw)
    v_ref = x[:, (Hq + Hkv) * D:width].reshape(T, Hkv, D)
    close(q_out, q_ref, dtype)
    pool = d["pool"].double().cpu()
    touched = torch.zeros(pool.shape[0], 64, dtype=torch.bool)
    for t in range(T):
        s, p = int(pg.seq_of[t]), int(pg.pos[t])
        page, r = int(pg.table[s, p // 64]), p % 64
        close(pool[page, 0, :, r], k_ref[t], dtype)
        close(pool[page, 1, :, r], v_ref[t], dtype)
        touched[page, r] = True
    same = (d["pool"] == before).all(-1).all(1).all(1).cpu()       # [pages, 64]
    assert same[~touched].all(), "a cache row of another position was written"
    if pairs < D // 2:      # the unrotated tail passes through: pair i is (i, i + D/2), not neighbours
        tail = rms_norm(x[:, :Hq * D].reshape(T, Hq, D), qw.double().cpu(), eps)[..., pairs:D // 2]
        close(q_out[..., pairs:D // 2], tail, dtype)


@pytest.mark.parametrize("M,D,pairs,Hq,Hkv,K,gate_rows,norm,rotate,write_kv", [
    (8, 64, 32, 32, 8, 2048, 32, True, True, True),        # the 1.2B shape: sixteen loads a round, clusters of four
    (3, 32, 10, 4, 2, 96, 0, True, True, True),            # predicated loads, clusters of two, partial rotation
    (13, 128, 64, 6, 3, 256, 16, False, True, True),       # 16-row instance, clusters of eight, no norm
    (5, 64, 32, 8, 2, 1024, 0, True, False, True),         # no rotation
    (8, 64, 20, 8, 4, 1024, 16, True, True, False)])       # a reader of another layer's cache: queries only
def test_gemm_small_m_with_the_rotation_behind_it(M, D, pairs, Hq, Hkv, K, gate_rows, norm, rotate, write_kv):
    """An attention layer's q/k/v product of a decode step with the per-head norm, the rotation and the cache write in
    its own kernel (the CTAs of a head as one cluster), against a float64 restatement; the columns behind the heads come
    out as the plain product leaves them, and no cache row of another position is touched."""
    lib = ops()
    starts = [3 + 67 * i for i in range(M)]
    pg = Paged(starts, [1] * M, Hq, Hkv, D, "bfloat16")
    pg.fill_pool(upto_start_only=True)
    d = pg.dev()
    width = (Hq + (2 * Hkv if write_kv else 0)) * D
    N = width + gate_rows
    g = torch.Generator(device="cpu").manual_seed(M * D + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K) * 3).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV) if K == 96 else None
    qw = (torch.rand(D, generator=g) + 0.5).to(DEV) if norm else None
    kw = (torch.rand(D, generator=g) + 0.5).to(DEV) if norm else None
    eps, theta = 1e-6, 10000.0
    inv = torch.zeros(D // 2, dtype=torch.float64)
    inv[:pairs] = (1.0 / theta ** (2.0 * torch.arange(pairs, dtype=torch.float64) / D)).float().double()
    ang = torch.arange(1024, dtype=torch.float64)[:, None] * inv[None, :]
    rope = torch.stack([ang.cos(), ang.sin()], -1).float().to(DEV) if rotate else None
    q_out = torch.full((M, Hq, D), float("nan"), device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    before = d["pool"].clone()
    lib.gemm_small_m_rope(x, w, out, bias, q_out, d["pool"] if write_kv else None, d["table"] if write_kv else None,
                          d["seq_of"], d["pos"], qw, kw, rope, Hq, Hkv, D, 64, eps)
    plain = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    lib.gemm_small_m(x, w, plain, bias)
    assert torch.equal(out, plain), "the product's own output changed"
    y = plain.double().cpu()
    pos = torch.tensor(pg.pos)

    def norm_rope(v, wt):     # v [M, heads, D]
        if wt is not None:
            v = rms_norm(v, wt.double().cpu(), eps)
        if not rotate:
            return v
        c, s_ = ang[pos].cos()[:, None, :], ang[pos].sin()[:, None, :]
        a, b = v[..., :D // 2], v[..., D // 2:]
        return torch.cat([a * c - b * s_, b * c + a * s_], -1)

    close(q_out, norm_rope(y[:, :Hq * D].reshape(M, Hq, D), qw), "bfloat16")
    if not write_kv:
        assert torch.equal(d["pool"], before)
        return
    k_ref = norm_rope(y[:, Hq * D:(Hq + Hkv) * D].reshape(M, Hkv, D), kw)
    v_ref = y[:, (Hq + Hkv) * D:width].reshape(M, Hkv, D)
    pool = d["pool"].double().cpu()
    touched = torch.zeros(pool.shape[0], 64, dtype=torch.bool)
    for t in range(M):
        s_, p_ = int(pg.seq_of[t]), int(pg.pos[t])
        page, r = int(pg.table[s_, p_ // 64]), p_ % 64
        close(pool[page, 0, :, r], k_ref[t], "bfloat16")
        assert torch.equal(pool[page, 1, :, r], v_ref[t]), "values are copied as they are"
        touched[page, r] = True
    same = (d["pool"] == before).all(-1).all(1).all(1).cpu()
    assert same[~touched].all(), "a cache row of another position was written"


# ------------------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K", [(96, 3), (200, 4), (64, 7), (40, 2), (72, 8), (48, 6)])
def test_short_conv_in_steps_equals_one_pass(dtype, H, K):
    """Three sequences fed in pieces of different sizes (one of them 5, 1, 1, 3, 2 as in the reference's
    tests/unit/backend/recurrent_ops_cases.h:89-118) give what one pass over each whole sequence gives,
    and never read a neighbour's tokens."""
    lib = ops()
    cuts = [[5, 1, 1, 3, 2], [1, 1, 9, 1], [12]]
    totals = [sum(c) for c in cuts]
    bcx_all = [(torch.randn(n, 3 * H + 8) * 2).to(DT[dtype]) for n in totals]
    taps = torch.randn(H, K)
    bias = torch.randn(H)
    w_t = taps.t().contiguous().to(DEV)
    n_slots = 5
    slots = [3, 0, 4]
    state = (torch.randn(n_slots, K - 1, H, device=DEV) * 40).to(DT[dtype])     # other slots' rows stay untouched
    lib.zero_rows(state, torch.tensor(slots, dtype=torch.int32, device=DEV))
    guard = state[[1, 2]].clone()

    def reference(s):
        x = bcx_all[s].double()
        B, C, X = x[:, :H], x[:, H:2 * H], x[:, 2 * H:3 * H]
        g = (B * X).to(DT[dtype]).double()                  # kept in the activation type, as the state keeps it
        ext = torch.cat([torch.zeros(K - 1, H, dtype=torch.float64), g], 0)
        conv = sum(taps[:, j].double()[None, :] * ext[j:j + x.shape[0]] for j in range(K)) + bias.double()
        return C * conv

    got = [torch.empty(n, H, device=DEV, dtype=DT[dtype]) for n in totals]
    at = [0, 0, 0]
    for step in range(max(len(c) for c in cuts)):
        part = [s for s in range(3) if step < len(cuts[s])]
        lens = [cuts[s][step] for s in part]
        bcx = torch.cat([bcx_all[s][at[s]:at[s] + n] for s, n in zip(part, lens)], 0).to(DEV)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
        seq_of = torch.tensor(np.repeat(np.arange(len(part)), lens), dtype=torch.int32, device=DEV)
        sl = torch.tensor([slots[s] for s in part], dtype=torch.int32, device=DEV)
        out = torch.empty(sum(lens), H, device=DEV, dtype=DT[dtype])
        lib.short_conv(bcx[:, :3 * H], w_t, bias.to(DEV), state, seq_of, cu, sl, out, all_single=all(n == 1 for n in lens))
        o = 0
        for s, n in zip(part, lens):
            got[s][at[s]:at[s] + n] = out[o:o + n]
            at[s] += n
            o += n
    for s in range(3):
        close(got[s], reference(s), dtype, factor=4)
    assert torch.equal(state[[1, 2]], guard)
    # the wrong tap order must not match: w[c, K-1] multiplies the current token
    x = bcx_all[2].double()
    g = (x[:, :H] * x[:, 2 * H:3 * H])
    ext = torch.cat([torch.zeros(K - 1, H, dtype=torch.float64), g], 0)
    flipped = x[:, H:2 * H] * (sum(taps[:, K - 1 - j].double()[None, :] * ext[j:j + 12] for j in range(K)) + bias.double())
    assert (got[2].double().cpu() - flipped).abs().max() > 0.5


@pytest.mark.parametrize("H,steps", [(1024, [[900, 3, 1, 1499], [1201, 2, 6, 1000]]),          # runs of 4 tokens
                                     (2048, [[2101, 5, 1, 299], [17, 2, 2300, 101]])])           # runs of 8 tokens
@pytest.mark.parametrize("K", [2, 3, 4, 5, 7, 8])
def test_short_conv_long_prompts(K, H, steps):
    """Long ragged prompts take the kernel in which a thread walks several tokens: sequences that start inside
    a thread's run, a run that ends past the last token, and a second step that continues from the state."""
    lib = ops()
    totals = [sum(st[s] for st in steps) for s in range(4)]
    bcx_all = [(torch.randn(n, 3 * H) * 2).to(torch.bfloat16) for n in totals]
    taps, bias = torch.randn(H, K), torch.randn(H)
    w_t = taps.t().contiguous().to(DEV)
    slots = [2, 0, 5, 3]
    state = (torch.randn(6, K - 1, H, device=DEV) * 40).to(torch.bfloat16)
    lib.zero_rows(state, torch.tensor(slots, dtype=torch.int32, device=DEV))
    guard = state[[1, 4]].clone()
    got = [torch.empty(n, H, device=DEV, dtype=torch.bfloat16) for n in totals]
    at = [0, 0, 0, 0]
    for lens in steps:
        bcx = torch.cat([bcx_all[s][at[s]:at[s] + n] for s, n in enumerate(lens)], 0).to(DEV)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
        seq_of = torch.tensor(np.repeat(np.arange(4), lens), dtype=torch.int32, device=DEV)
        out = torch.full((sum(lens), H), float("nan"), device=DEV, dtype=torch.bfloat16)
        lib.short_conv(bcx, w_t, bias.to(DEV), state, seq_of, cu, torch.tensor(slots, dtype=torch.int32, device=DEV), out)
        o = 0
        for s, n in enumerate(lens):
            got[s][at[s]:at[s] + n] = out[o:o + n]
            at[s] += n
            o += n
    for s in range(4):
        x = bcx_all[s].double()
        g = (x[:, :H] * x[:, 2 * H:]).to(torch.bfloat16).double()
        ext = torch.cat([torch.zeros(K - 1, H, dtype=torch.float64), g], 0)
        conv = sum(taps[:, j].double()[None, :] * ext[j:j + x.shape[0]] for j in range(K)) + bias.double()
        close(got[s], x[:, H:2 * H] * conv, "bfloat16", factor=4)
    assert torch.equal(state[[1, 4]], guard)


def test_argmax_ties_and_width():
    lib = ops()
    V = 65536 + 77
    logits = torch.randn(5, V, device=DEV)
    logits[0, 40000] = 50.0
    logits[1, V - 1] = 50.0
    logits[2, 9] = 50.0
    logits[2, 70] = 50.0          # a tie: the lower index wins
    logits[3, :] = -1.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    lib.argmax(logits, out)
    assert out.tolist()[:4] == [40000, V - 1, 9, 0] and out[4].item() == int(logits[4].argmax())
