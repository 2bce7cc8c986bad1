"""What the parts share on one device: the precision mode, scratch buffers, matrix products.

Two modes. "bfloat16": matrices, activations between kernels and the cache are bfloat16;
norm weights, the residual stream, softmax, rotation tables and logits are float32.
"float32": everything is float32 and every matrix product runs on CUDA-core FMAs (no
tensor cores, no TF32), slower but exact enough to show what bfloat16 hides.

Matrix products: the float32 mode uses this library's own kernel for every shape. The
bfloat16 mode uses this library's kernels where the reference uses its own (products with
few rows, src/backend/sycl/sycl_kernels.cpp:630-714, `kGemvMaxRows`) and the vendor's
GEMM library where the reference calls one (prefill-sized products, oneMKL there,
src/backend/sycl/sycl_matmul.cpp:44-110; cuBLAS through torch.mm here).
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from ..ops import lib as ops

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "f32": torch.float32}


class Workspace:
    """Named scratch buffers that grow to the largest request and are then reused.
    A name is used by one producer at a time; layers run one after another and share them."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple, torch.Tensor] = {}      # (name, dtype, shape) -> the view handed out last time
        self.frozen = False

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= s
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"scratch buffer '{name}' would have to grow after it was frozen")
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:     # views of the old buffer
                del self._views[k]
        view = buf[:n].view(*shape)
        if len(self._views) < 4096:
            self._views[(name, dtype, shape)] = view
        return view


class Runtime:
    def __init__(self, dtype: str = "bfloat16", device="cuda:0"):
        if dtype not in DTYPES:
            raise ValueError(f"dtype '{dtype}' is not supported (bfloat16, float32 are)")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        self.act_dtype = DTYPES[dtype]
        self.mode = "bfloat16" if self.act_dtype == torch.bfloat16 else "float32"
        self.ws = Workspace(self.device)
        self.shared: Dict[Tuple, object] = {}     # parts memoise what equal specs can share (tables)
        # cuBLAS may otherwise reduce split products in bfloat16
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        # decode attention cuts each sequence's keys over enough CTAs to fill this many CTA slots an SM
        # (0: sized by rounds of CTAs, parts/attention.py decode_splits; n > 0: n CTAs an SM, the earlier rule)
        self.attn_split_factor = int(os.environ.get("XS_ATTN_SPLIT_FACTOR", "0"))
        self.attn_fixed_cost = float(os.environ.get("XS_ATTN_FIXED_COST", "2"))
        # attention of prompts: "tcgen05" (head size 64 and groups that divide 128; everything else takes the
        # mma.sync kernel anyway) or "mma". Measured on B200, 32 heads over 8: 2,048 tokens 62 against 97 us,
        # 2,048 tokens after 30,000: 1.01 against 1.87 ms.
        self.prompt_attention = os.environ.get("XS_PROMPT_ATTENTION", "tcgen05")
        if self.prompt_attention not in ("tcgen05", "mma"):
            raise ValueError("XS_PROMPT_ATTENTION must be 'tcgen05' or 'mma'")
        # Products with at most `small_m` rows use this library's weight-streaming kernel (it takes up to 16), and so do,
        # up to `narrow_m` rows, the products whose outputs are at most `narrow_n` columns wide (few_rows_shape below
        # has the measurements). The reference draws one line: its own gemv up to 8 rows, the vendor's library above
        # (src/backend/sycl/sycl_kernels.h:280).
        self.small_m = int(os.environ.get("XS_SMALL_M", "8"))
        if not 0 <= self.small_m <= 16:
            raise ValueError("XS_SMALL_M must be 0 to 16")
        self.narrow_m = int(os.environ.get("XS_NARROW_M", "16"))
        if not 0 <= self.narrow_m <= 16:
            raise ValueError("XS_NARROW_M must be 0 to 16")
        self.narrow_n = int(os.environ.get("XS_NARROW_N", "8192"))
        # decode: RMSNorm carried by the products on either side of it instead of a kernel of its own
        self.fuse_norms = os.environ.get("XS_NO_NORM_FUSION", "0") != "1"
        # Products with more rows. "auto": this library's tcgen05 kernel where it fuses an epilogue that the
        # library product cannot (the gate/up product with its activation, from 512 tokens on: measured on
        # B200 at 2,048 tokens, 99 us against 95 us and a separate activation pass over 100 MB), cuBLAS elsewhere
        # (in_proj, out_proj, qkv and the down projection run 12 to 45 % faster there at 2,048 tokens, mostly
        # because it cuts the last, partly filled wave of tiles finer). "tcgen05": every such product on this
        # library's kernel. "library": none.
        self.many_rows = os.environ.get("XS_MANY_ROWS_GEMM", "auto")
        if self.many_rows not in ("auto", "library", "tcgen05"):
            raise ValueError("XS_MANY_ROWS_GEMM must be 'auto', 'library' or 'tcgen05'")
        self.fused_from_rows = 512
        ops.load()
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.gemm_scratch = torch.zeros(8 * 1024 * 1024, dtype=torch.uint8, device=self.device)
        # Work done behind its producer inside the producer's kernel. XS_TAILS names what runs so (a comma list of
        # conv, attn, argmax, rope), the rest stay kernels of their own; XS_NO_TAILS=1: none. Each tail of the few-row
        # product is a kernel instance of its own: with the tails' code in every instance, the products without a
        # tail carried its registers and the whole step took 0.642 instead of 0.628 ms. Measured on B200, 1.2B shape,
        # decode at batch 8:
        #   conv    the short convolution behind in_proj, by the three CTAs of a group of channels as one thread-block
        #           cluster that meets in shared memory: 0.650 -> 0.642 ms a step (when the three still met through
        #           global memory and a counter it cost 17 us instead)
        #   attn    the merge of decode attention's key splits by the CTA of a (sequence, kv head) that stores last:
        #           the same time with six launches fewer
        #   argmax  behind the head product through atomics on one word: +8 us, off
        #   rope    an attention layer's per-head norms, rotation and cache write behind its q/k/v product, the CTAs
        #           of a head as one cluster: +10 us, off
        # The zeroed words below are what the counting tails count in and leave zeroed.
        self.fuse_tails = os.environ.get("XS_NO_TAILS", "0") != "1"
        tails = os.environ.get("XS_TAILS", "conv,attn").split(",")
        self.tail_conv, self.tail_attn, self.tail_argmax = ["conv" in tails, "attn" in tails, "argmax" in tails]
        self.tail_rope = "rope" in tails
        self.conv_counters = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self.attn_counters = torch.zeros(65536, dtype=torch.int32, device=self.device)
        self.amax_keys = torch.zeros(16, dtype=torch.int64, device=self.device)
        self.amax_counter = torch.zeros(1, dtype=torch.int32, device=self.device)

    # -------------------------------------------------------------- weights
    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix or table in the mode's element type, on the device."""
        return t.to(device=self.device, dtype=self.act_dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights, taps and biases stay float32 in both modes."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    # ------------------------------------------------------ matrix products
    def few_rows_shape(self, rows: int, w: torch.Tensor) -> bool:
        """Whether a product of `rows` rows with the weight w goes to the library's own weight-streaming kernel."""
        # up to `small_m` rows: every product. Up to `narrow_m` rows: the products with narrow outputs, where the
        # library's kernels leave most SMs idle (measured on B200 at 9 to 16 rows, us, this kernel against the
        # library: N 2048 K 2048 2.9 to 3.0 against 5.1; N 3072 K 2048 3.5 to 3.6 against 5.4; N 2048 K 8192
        # 10.9 to 11.2 against 12.7; N 6144 K 2048 6.8 to 7.0 against 7.2; but N 16384 K 2048 15.3 to 16.2 against
        # 13.0 and N 65536 46 to 50 against 42)
        return self.mode == "bfloat16" and (rows <= self.small_m or (rows <= self.narrow_m and w.shape[0] <= self.narrow_n))

    def few_rows(self, x, w: torch.Tensor) -> bool:
        """Whether this product goes to the library's own weight-streaming kernel."""
        x = getattr(x, "x", x)      # a Prenormed input counts as its tensor
        return (self.few_rows_shape(x.shape[0], w)
                and ops.gemm_small_m_supports(x.shape[0], x.shape[1], x.stride(0), w.stride(0)))

    def tensor_core_product(self, x: torch.Tensor, w: torch.Tensor, fused: bool = False) -> bool:
        """Whether this product goes to the library's tcgen05 kernel. `fused`: the caller would use an
        epilogue of that kernel that saves a pass over the output."""
        if self.mode != "bfloat16" or self.many_rows == "library" or hasattr(x, "ssq"):
            return False
        if self.many_rows == "auto" and not (fused and x.shape[0] >= self.fused_from_rows):
            return False
        return ops.gemm_tc_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))

    def few_rows_product(self, x, w, out, bias=None, swiglu: bool = False, residual=None, next_w=None, next_x=None,
                         out_ssq=None, conv=None, argmax_into=None) -> None:
        """The library's weight-streaming product, with K cut over several CTAs where the output is
        narrow; the partial sums meet in one zero-initialised scratch buffer that lives as long as
        the runtime (its tail holds the kernel's counters). `x` may be a Prenormed input; `residual`
        (the float32 stream) takes the result instead of `out`, with `next_*` / `out_ssq` as in
        ops.gemm_small_m."""
        norm = {}
        if hasattr(x, "ssq"):
            norm = dict(in_ssq=x.ssq, in_width=x.width, in_eps=x.eps)
            x = x.x
        ksplit = ops.gemm_small_m_ksplit(x.shape[0], w.shape[0], x.shape[1], self.sm_count)
        if ksplit > 1 and ops.gemm_small_m_scratch_bytes(x.shape[0], w.shape[0], ksplit) > self.gemm_scratch.numel():
            ksplit = 1
        if conv is not None:
            ksplit = 1          # the convolution behind the product counts whole tiles
            conv = dict(conv, counters=self.conv_counters)
        ops.gemm_small_m(x, w, out, bias, residual=residual, swiglu=swiglu, ksplit=ksplit,
                         scratch=self.gemm_scratch if ksplit > 1 else None, next_w=next_w, next_x=next_x, out_ssq=out_ssq,
                         conv=conv, argmax=None if argmax_into is None else (argmax_into, self.amax_keys, self.amax_counter),
                         **norm)

    def rope_behind_product(self, x, w, head_dim: int) -> bool:
        """Whether an attention layer's per-head norm, rotation and cache write (one token a sequence) can run behind
        its q/k/v product in the product's kernel."""
        return (self.fuse_tails and self.tail_rope and self.few_rows(x, w) and head_dim in (32, 64, 128)
                and w.shape[0] % 16 == 0)

    def few_rows_rope(self, x, w, out, bias, **rope) -> None:
        """ops.gemm_small_m_rope; `x` may be a Prenormed input."""
        norm = {}
        if hasattr(x, "ssq"):
            norm = dict(in_ssq=x.ssq, in_width=x.width, in_eps=x.eps)
            x = x.x
        ops.gemm_small_m_rope(x, w, out, bias, **rope, **norm)

    def conv_behind_product(self, x, w, channels: int) -> bool:
        """Whether a short convolution of one token a sequence can run in the tail of its in_proj product."""
        # (up to 8 rows: at 9 to 16 the kernel of its own is the faster way, 0.819 against 0.830 ms a step at batch 12)
        rows = getattr(x, "x", x).shape[0]
        return (self.fuse_tails and self.tail_conv and rows <= 8 and self.few_rows(x, w) and channels % 16 == 0
                and channels // 16 <= self.conv_counters.numel() and w.shape[0] == 3 * channels)

    def linear(self, x: torch.Tensor, w: torch.Tensor, name: str, bias: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, argmax_into: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x[M, K] . w[N, K]^T (+ bias) into the scratch buffer `name`. x may be a Prenormed input. `argmax_into`
        (int32 [M]) also takes each row's column of the largest output, behind the product where the few-row kernel
        runs it, by the argmax kernel otherwise."""
        M, N = x.shape[0], w.shape[0]
        if argmax_into is not None:
            if self.mode == "bfloat16" and self.fuse_tails and self.tail_argmax and M <= 16 and self.few_rows(x, w):
                out = self.ws.get(name, (M, N), out_dtype or self.act_dtype)
                self.few_rows_product(x, w, out, bias, argmax_into=argmax_into)
                return out
            out = self.linear(x, w, name, bias, out_dtype)
            ops.argmax(out, argmax_into)
            return out
        if hasattr(x, "ssq") and not self.few_rows(x, w):
            raise RuntimeError("a Prenormed input needs the few-row product")
        out_dtype = out_dtype or self.act_dtype
        out = self.ws.get(name, (M, N), out_dtype)
        if self.mode == "float32":
            ops.gemm_generic(x, w, out, bias)
        elif self.few_rows(x, w):
            self.few_rows_product(x, w, out, bias)
        elif self.tensor_core_product(x, w):
            ops.gemm_tc(x, w, out, bias)
        elif bias is not None:
            # (the library product has no float32 bias: this library's tensor-core kernel adds it in its epilogue)
            if (self.many_rows != "library" and not hasattr(x, "ssq")
                    and ops.gemm_tc_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))):
                ops.gemm_tc(x, w, out, bias)
            else:
                ops.gemm_generic(x, w, out, bias)
        elif out_dtype == torch.float32:
            out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
        else:
            torch.mm(x, w.t(), out=out)
        return out
