// Flash-style attention over the paged bfloat16 cache on tensor cores, for prefill and decode.
//
// One CTA (4 warps) owns a tile of 64 query rows that share one kv head: rows are
// (token, head of the group) pairs, row r = token r / G, head r % G with G = heads / kv_heads,
// so keys and values are read once for the whole group. It walks the cache in blocks of
// 64 keys (one page: 64 x head_dim contiguous elements for keys, the same for values),
// double-buffered with cp.async, S = Q K^T and O += P V with mma.sync m16n8k16 (bfloat16 in,
// float32 accumulate), softmax online in float32 (base-2 exponentials of scores pre-multiplied
// by scale * log2 e). Query at position pos sees key j iff j <= pos and (window == 0 or
// pos - j < window) (src/backend/cpu_ref/ops.cpp:567-571). Rows of keys and values past the
// sequence's length are zero-filled in shared memory, so stale cache contents never reach
// the arithmetic.
//
// When a tile's key range is split over several CTAs (decode: few tiles, long ranges), each
// writes an unnormalised partial (O, running max, running sum) to scratch and
// attention_combine_kernel merges them; this is the reference's attention_rows +
// attention_combine pair (src/backend/sycl/sycl_kernels.h:223-244), and its XMX flash kernel
// for prefill (src/backend/sycl/sycl_flash_attention.cpp:1-15), as one kernel.
//
// Head sizes: multiples of 16 up to 128 that are instantiated below; others are refused here
// and served by the generic kernel.
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BM = 64;       // query rows per CTA
constexpr int BN = 64;       // keys per block = page size
constexpr int NTHREADS = 128;

struct AttnParams {
    const __nv_bfloat16* q;          // [T, Hq, D]
    const __nv_bfloat16* pool;       // [pages, 2, Hkv, 64, D]
    const int32_t* page_table;       // [n_seqs, P]
    int P;
    const int32_t* cu_seqlens;       // [n_seqs + 1]
    const int32_t* kv_lens;          // [n_seqs] length after this step
    const __nv_bfloat16* gate;       // [T, ld_gate] gate logits or null
    int64_t ld_gate;
    __nv_bfloat16* out;              // [T, Hq, D]
    float* part_o;                   // [T * Hq, splits, D]
    float* part_ml;                  // [T * Hq, splits, 2]
    int Hq, Hkv, G, tokens_per_tile, window, splits;
    int prefetch_blocks;             // decode: how many of a CTA's first key blocks are hinted into L2 before the wait
    int decode_rows;                 // every tile has at most 16 rows: the warps split the keys instead
    float scale_log2;
    unsigned int* counters;          // decode with key splits: one zeroed word per (sequence, kv head), left zeroed; or null
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (2 ulp; -inf gives 0): the softmax weights are rounded to bfloat16 anyway
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int NST>
__global__ void __launch_bounds__(NTHREADS, (D <= 64 ? 4 : 2)) attention_mma_kernel(const AttnParams p) {
    constexpr int LD = D + 8;              // padded row: ldmatrix reads 8 rows without bank conflicts
    constexpr int KSTEPS = D / 16;         // k-steps of Q K^T
    constexpr int DTILES = D / 8;          // n-tiles of the output
    constexpr int CHUNKS = D / 8;          // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* k_sm = q_sm + BM * LD;            // [NST][BN][LD]
    __nv_bfloat16* v_sm = k_sm + NST * BN * LD;      // [NST][BN][LD]

    pdl_launch_dependents();
    pdl_wait();
    // later tiles see more keys: they are started first, so that the short ones fill the tail
    const int tile = gridDim.x - 1 - blockIdx.x, seq = blockIdx.y;
    const int kvh = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int tok_begin = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - tok_begin;
    const int t0 = tile * p.tokens_per_tile;
    if (t0 >= q_len) return;
    const int nt = min(p.tokens_per_tile, q_len - t0);
    const int kv_len = p.kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;
    const int hi = pos0 + nt;                                     // keys [lo, hi) matter to this tile
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int b_lo = lo / BN, nb = (hi + BN - 1) / BN - b_lo;
    const int bs = b_lo + (int)((int64_t)nb * split / p.splits);
    const int be = b_lo + (int)((int64_t)nb * (split + 1) / p.splits);
    const int32_t* table = p.page_table + (int64_t)seq * p.P;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.G;
    const int rows_valid = nt * G;
    const bool warp_active = warp * 16 < rows_valid;

    // ---- Q tile: row r = (token t0 + r / G, head kvh * G + r % G); invalid rows are zero
    for (int c = threadIdx.x; c < BM * CHUNKS; c += NTHREADS) {
        const int r = c / CHUNKS, ch = c % CHUNKS;
        const bool ok = r < rows_valid;
        const int ti = ok ? r / G : 0, g = ok ? r % G : 0;
        const __nv_bfloat16* src = p.q + ((int64_t)(tok_begin + t0 + ti) * p.Hq + kvh * G + g) * D + ch * 8;
        cp_async16(q_sm + r * LD + ch * 8, src, ok);
    }
    auto load_block = [&](int b, int stage) {
        const int page = table[b];
        const int page_at = max(page, 0);      // a page given back (-1) is never read: its rows are zero-filled
        const __nv_bfloat16* kbase = p.pool + (((int64_t)page_at * 2 + 0) * p.Hkv + kvh) * BN * D;
        const __nv_bfloat16* vbase = p.pool + (((int64_t)page_at * 2 + 1) * p.Hkv + kvh) * BN * D;
        __nv_bfloat16* ks = k_sm + stage * BN * LD;
        __nv_bfloat16* vs = v_sm + stage * BN * LD;
        for (int c = threadIdx.x; c < BN * CHUNKS; c += NTHREADS) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const bool ok = page >= 0 && b * BN + r < hi;
            cp_async16(ks + r * LD + ch * 8, kbase + (ok ? r * D + ch * 8 : 0), ok);
            cp_async16(vs + r * LD + ch * 8, vbase + (ok ? r * D + ch * 8 : 0), ok);
        }
    };
    // NST - 1 blocks are requested before the first is used; one commit group per block, empty ones too,
    // so that "all but the newest NST - 2 groups have landed" always means "block b is here"
#pragma unroll
    for (int s = 0; s < NST - 1; ++s) {
        if (bs + s < be) load_block(bs + s, s);
        cp_async_commit();
    }

    // this thread's two rows and their positions (-1: no key is visible)
    const int r1 = warp * 16 + (lane >> 2), r2 = r1 + 8;
    const int pos1 = r1 < rows_valid ? pos0 + r1 / G : -1;
    const int pos2 = r2 < rows_valid ? pos0 + r2 / G : -1;

    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
    unsigned qf[KSTEPS][4];
    bool q_loaded = false;

    for (int b = bs, it = 0; b < be; ++b, ++it) {
        const int stage = it % NST;
        cp_async_wait<NST - 2>();
        __syncthreads();            // block b has landed for everyone, and everyone is done with block b - 1
        if (b + NST - 1 < be) load_block(b + NST - 1, (it + NST - 1) % NST);   // into the stage block b - 1 used
        cp_async_commit();
        if (warp_active) {
            if (!q_loaded) {
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk)
                    ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3],
                                q_sm + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
                q_loaded = true;
            }
            const __nv_bfloat16* ks = k_sm + stage * BN * LD;
            const __nv_bfloat16* vs = v_sm + stage * BN * LD;
            float s[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int np = 0; np < BN / 16; ++np) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3,
                                ks + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(s[2 * np], qf[kk], b0, b1);
                    mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
                }
            }
            // scale, mask, running max. A block that every row of the tile sees whole (all of it at or before
            // the tile's first position and inside every row's window) needs no per-element test.
            const int key0 = b * BN + (lane & 3) * 2;
            const bool whole = b * BN + BN - 1 <= pos0 && (p.window == 0 || pos0 + nt - 1 - b * BN < p.window);
            float mx1 = -INFINITY, mx2 = -INFINITY;
            if (whole) {
#pragma unroll
                for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        s[i][e] = pos1 >= 0 ? s[i][e] * p.scale_log2 : -INFINITY;
                        s[i][2 + e] = pos2 >= 0 ? s[i][2 + e] * p.scale_log2 : -INFINITY;
                        mx1 = fmaxf(mx1, s[i][e]);
                        mx2 = fmaxf(mx2, s[i][2 + e]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + i * 8 + e;
                        const bool v1 = key <= pos1 && (p.window == 0 || pos1 - key < p.window);
                        const bool v2 = key <= pos2 && (p.window == 0 || pos2 - key < p.window);
                        s[i][e] = v1 ? s[i][e] * p.scale_log2 : -INFINITY;
                        s[i][2 + e] = v2 ? s[i][2 + e] * p.scale_log2 : -INFINITY;
                        mx1 = fmaxf(mx1, s[i][e]);
                        mx2 = fmaxf(mx2, s[i][2 + e]);
                    }
                }
            }
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 1));
            mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 2));
            const float mn1 = fmaxf(m1, mx1), mn2 = fmaxf(m2, mx2);
            const float base1 = mn1 == -INFINITY ? 0.0f : mn1, base2 = mn2 == -INFINITY ? 0.0f : mn2;
            const float c1 = fast_exp2(m1 - base1), c2 = fast_exp2(m2 - base2);   // 0 while nothing was seen
            m1 = mn1;
            m2 = mn2;
            l1 *= c1;
            l2 *= c2;
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
                o[i][0] *= c1;
                o[i][1] *= c1;
                o[i][2] *= c2;
                o[i][3] *= c2;
            }
            unsigned pf[BN / 16][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
                const float p0 = fast_exp2(s[i][0] - base1), p1 = fast_exp2(s[i][1] - base1);
                const float p2 = fast_exp2(s[i][2] - base2), p3 = fast_exp2(s[i][3] - base2);
                l1 += p0 + p1;
                l2 += p2 + p3;
                pf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
                pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3,
                                      vs + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + dp * 16 + (lane >> 4) * 8);
                    mma_bf16(o[2 * dp], pf[kk], b0, b1);
                    mma_bf16(o[2 * dp + 1], pf[kk], b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (!warp_active) return;

    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    l2 += __shfl_xor_sync(0xffffffffu, l2, 1);
    l2 += __shfl_xor_sync(0xffffffffu, l2, 2);

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half == 0 ? r1 : r2;
        if (r >= rows_valid) continue;
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const float l = half == 0 ? l1 : l2, m = half == 0 ? m1 : m2;
        const int64_t row = (int64_t)t * p.Hq + h;
        if (p.splits == 1) {
            float f = l > 0.0f ? 1.0f / l : 0.0f;
            if (p.gate != nullptr) f *= 1.0f / (1.0f + __expf(-__bfloat162float(p.gate[(int64_t)t * p.ld_gate + h])));
            __nv_bfloat16* dst = p.out + row * D + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < DTILES; ++i)
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) =
                    __floats2bfloat162_rn(o[i][half * 2] * f, o[i][half * 2 + 1] * f);
        } else {
            float* dst = p.part_o + (row * p.splits + split) * D + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < DTILES; ++i)
                *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
            if ((lane & 3) == 0) {
                p.part_ml[(row * p.splits + split) * 2 + 0] = m;
                p.part_ml[(row * p.splits + split) * 2 + 1] = l;
            }
        }
    }
}

// Decoding (at most 16 query rows a tile: one token's group of heads): the rows would keep a single warp
// busy, so here the four warps split every 64-key block instead, 16 keys each, each with its own
// running maximum, sum and output; they are merged through shared memory at the end. Everything else
// (paging, masks, splits, zero-filled tails) is as in the kernel above.
template <int D, int NST>
__global__ void __launch_bounds__(NTHREADS) attention_decode_mma_kernel(const AttnParams p) {
    constexpr int LD = D + 8;
    constexpr int KSTEPS = D / 16;
    constexpr int DTILES = D / 8;
    constexpr int CHUNKS = D / 8;
    constexpr int QROWS = 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [16][LD]
    __nv_bfloat16* k_sm = q_sm + QROWS * LD;                             // [NST][BN][LD]
    __nv_bfloat16* v_sm = k_sm + NST * BN * LD;                          // [NST][BN][LD]
    __shared__ float sm_m[4][QROWS], sm_l[4][QROWS];
    __shared__ int pages_sm[64];

    pdl_launch_dependents();
    // The step's description (lengths, page table) was copied to the device before the step began, and cached
    // keys and values of earlier positions do not change during a step: the first blocks of this CTA's share of
    // the cache are asked into L2 before waiting for the kernel that writes the current position's keys and
    // values. Only the first: hints for a whole long share (hundreds of MB over all CTAs) push one another out of
    // L2 and the cache is then read from memory twice (64 sequences of 1k to 24k keys: 483 us with the whole share
    // hinted, 308 us with two blocks).
    const int seq = blockIdx.y;
    const int kvh = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int tok_begin = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - tok_begin;
    const int t0 = blockIdx.x * p.tokens_per_tile;
    if (t0 >= q_len) return;
    const int nt = min(p.tokens_per_tile, q_len - t0);
    const int kv_len = p.kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;
    const int hi = pos0 + nt;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int b_lo = lo / BN, nb = (hi + BN - 1) / BN - b_lo;
    const int bs = b_lo + (int)((int64_t)nb * split / p.splits);
    const int be = b_lo + (int)((int64_t)nb * (split + 1) / p.splits);
    const int32_t* table = p.page_table + (int64_t)seq * p.P;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.G;
    const int rows_valid = nt * G;          // <= 16
    {
        constexpr int kLines = BN * D * 2 / 128;          // 128-byte lines of one block of keys (or values)
        for (int b = bs; b < min(be, bs + p.prefetch_blocks); ++b) {
            const int page = table[b];
            if (page < 0) continue;
            const __nv_bfloat16* kbase = p.pool + (((int64_t)page * 2 + 0) * p.Hkv + kvh) * BN * D;
            const __nv_bfloat16* vbase = p.pool + (((int64_t)page * 2 + 1) * p.Hkv + kvh) * BN * D;
            for (int i = threadIdx.x; i < 2 * kLines; i += NTHREADS) {
                const __nv_bfloat16* at = (i < kLines ? kbase : vbase) + (i % kLines) * 64;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(at));
            }
        }
    }
    // this CTA's page numbers in one coalesced read (in pieces of 64 blocks); the first piece before the wait: the
    // page table is part of the step's description
    auto load_pages = [&](int from) {
        __syncthreads();
        if (threadIdx.x < 64 && from + (int)threadIdx.x < be) pages_sm[threadIdx.x] = table[from + threadIdx.x];
        __syncthreads();
    };
    int pages_from = bs;
    load_pages(pages_from);
    pdl_wait();

    for (int c = threadIdx.x; c < QROWS * CHUNKS; c += NTHREADS) {
        const int r = c / CHUNKS, ch = c % CHUNKS;
        const bool ok = r < rows_valid;
        const int ti = ok ? r / G : 0, g = ok ? r % G : 0;
        const __nv_bfloat16* src = p.q + ((int64_t)(tok_begin + t0 + ti) * p.Hq + kvh * G + g) * D + ch * 8;
        cp_async16(q_sm + r * LD + ch * 8, src, ok);
    }
    auto load_block = [&](int b, int stage) {
        const int page = pages_sm[b - pages_from];
        const int page_at = max(page, 0);
        const __nv_bfloat16* kbase = p.pool + (((int64_t)page_at * 2 + 0) * p.Hkv + kvh) * BN * D;
        const __nv_bfloat16* vbase = p.pool + (((int64_t)page_at * 2 + 1) * p.Hkv + kvh) * BN * D;
        __nv_bfloat16* ks = k_sm + stage * BN * LD;
        __nv_bfloat16* vs = v_sm + stage * BN * LD;
        for (int c = threadIdx.x; c < BN * CHUNKS; c += NTHREADS) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const bool ok = page >= 0 && b * BN + r < hi;
            cp_async16(ks + r * LD + ch * 8, kbase + (ok ? r * D + ch * 8 : 0), ok);
            cp_async16(vs + r * LD + ch * 8, vbase + (ok ? r * D + ch * 8 : 0), ok);
        }
    };
#pragma unroll
    for (int s = 0; s < NST - 1; ++s) {
        if (bs + s < be) load_block(bs + s, s);
        cp_async_commit();
    }

    const int r1 = lane >> 2, r2 = r1 + 8;
    const int pos1 = r1 < rows_valid ? pos0 + r1 / G : -1;
    const int pos2 = r2 < rows_valid ? pos0 + r2 / G : -1;
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
    unsigned qf[KSTEPS][4];
    bool q_loaded = false;

    for (int b = bs, it = 0; b < be; ++b, ++it) {
        const int stage = it % NST;
        cp_async_wait<NST - 2>();
        __syncthreads();
        const int nxt = b + NST - 1;
        if (nxt < be) {
            if (nxt - pages_from >= 64) {          // the page numbers held do not reach that far: refill (rare: > 4,096 keys a split)
                cp_async_wait<0>();
                pages_from = b;
                load_pages(pages_from);
            }
            load_block(nxt, (it + NST - 1) % NST);
        }
        cp_async_commit();
        if (!q_loaded) {
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk)
                ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], q_sm + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
            q_loaded = true;
        }
        const __nv_bfloat16* ks = k_sm + stage * BN * LD + warp * 16 * LD;     // this warp's 16 keys of the block
        const __nv_bfloat16* vs = v_sm + stage * BN * LD + warp * 16 * LD;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            unsigned b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, ks + ((lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[0], qf[kk], b0, b1);
            mma_bf16(s[1], qf[kk], b2, b3);
        }
        const int key0 = b * BN + warp * 16 + (lane & 3) * 2;
        float mx1 = -INFINITY, mx2 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + i * 8 + e;
                const bool v1 = key <= pos1 && (p.window == 0 || pos1 - key < p.window);
                const bool v2 = key <= pos2 && (p.window == 0 || pos2 - key < p.window);
                s[i][e] = v1 ? s[i][e] * p.scale_log2 : -INFINITY;
                s[i][2 + e] = v2 ? s[i][2 + e] * p.scale_log2 : -INFINITY;
                mx1 = fmaxf(mx1, s[i][e]);
                mx2 = fmaxf(mx2, s[i][2 + e]);
            }
        }
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 1));
        mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 2));
        const float mn1 = fmaxf(m1, mx1), mn2 = fmaxf(m2, mx2);
        const float base1 = mn1 == -INFINITY ? 0.0f : mn1, base2 = mn2 == -INFINITY ? 0.0f : mn2;
        const float c1 = fast_exp2(m1 - base1), c2 = fast_exp2(m2 - base2);
        m1 = mn1;
        m2 = mn2;
        l1 *= c1;
        l2 *= c2;
#pragma unroll
        for (int i = 0; i < DTILES; ++i) {
            o[i][0] *= c1;
            o[i][1] *= c1;
            o[i][2] *= c2;
            o[i][3] *= c2;
        }
        unsigned pf[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float p0 = fast_exp2(s[i][0] - base1), p1 = fast_exp2(s[i][1] - base1);
            const float p2 = fast_exp2(s[i][2] - base2), p3 = fast_exp2(s[i][3] - base2);
            l1 += p0 + p1;
            l2 += p2 + p3;
            pf[i * 2 + 0] = pack_bf16(p0, p1);
            pf[i * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            unsigned b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, vs + (((lane >> 3) & 1) * 8 + (lane & 7)) * LD + dp * 16 + (lane >> 4) * 8);
            mma_bf16(o[2 * dp], pf, b0, b1);
            mma_bf16(o[2 * dp + 1], pf, b2, b3);
        }
    }
    cp_async_wait<0>();
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    l2 += __shfl_xor_sync(0xffffffffu, l2, 1);
    l2 += __shfl_xor_sync(0xffffffffu, l2, 2);

    // ---- merge the four warps: their outputs go through the (now idle) key stages
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(k_sm);          // [4][16][D]
    if ((lane & 3) == 0) {
        sm_m[warp][r1] = m1;
        sm_l[warp][r1] = l1;
        sm_m[warp][r2] = m2;
        sm_l[warp][r2] = l2;
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
        float* d1 = sm_o + ((warp * QROWS + r1) * D) + i * 8 + (lane & 3) * 2;
        float* d2 = sm_o + ((warp * QROWS + r2) * D) + i * 8 + (lane & 3) * 2;
        d1[0] = o[i][0];
        d1[1] = o[i][1];
        d2[0] = o[i][2];
        d2[1] = o[i][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows_valid * D; idx += NTHREADS) {
        const int r = idx / D, d = idx % D;
        float m = fmaxf(fmaxf(sm_m[0][r], sm_m[1][r]), fmaxf(sm_m[2][r], sm_m[3][r]));
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = sm_m[w][r] == -INFINITY ? 0.0f : fast_exp2(sm_m[w][r] - m);
            l += sm_l[w][r] * f;
            acc += sm_o[(w * QROWS + r) * D + d] * f;
        }
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const int64_t row = (int64_t)t * p.Hq + h;
        if (p.splits == 1) {
            float f = l > 0.0f ? 1.0f / l : 0.0f;
            if (p.gate != nullptr) f *= 1.0f / (1.0f + __expf(-__bfloat162float(p.gate[(int64_t)t * p.ld_gate + h])));
            p.out[row * D + d] = __float2bfloat16_rn(acc * f);
        } else {
            p.part_o[(row * p.splits + split) * D + d] = acc;
            if (d == 0) {
                p.part_ml[(row * p.splits + split) * 2 + 0] = m;
                p.part_ml[(row * p.splits + split) * 2 + 1] = l;
            }
        }
    }
    if (p.splits == 1 || p.counters == nullptr) return;
    // ---- key splits without a kernel of their own to merge them: the CTA of a (sequence, kv head) that stores its part
    // last merges all of them (the same sums in the same order as attention_combine_kernel). Nobody waits for anybody.
    __shared__ bool is_last;
    __threadfence();
    __syncthreads();
    unsigned int* counter = p.counters + (int64_t)seq * p.Hkv + kvh;
    if (threadIdx.x == 0) is_last = atomicAdd(counter, 1u) == (unsigned)p.splits - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float* w_sm = reinterpret_cast<float*>(v_sm);            // [rows][splits] weights, then [rows] 1 / sum (times the gate)
    float* f_sm = w_sm + QROWS * 64;
    for (int r = warp; r < rows_valid; r += NTHREADS / 32) {           // a warp a row; lane s holds splits s and s + 32
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const float* ml = p.part_ml + ((int64_t)t * p.Hq + h) * p.splits * 2;
        const float ms0 = lane < p.splits ? __ldcg(ml + 2 * lane) : -INFINITY;
        const float ms1 = lane + 32 < p.splits ? __ldcg(ml + 2 * (lane + 32)) : -INFINITY;
        const float ls0 = lane < p.splits ? __ldcg(ml + 2 * lane + 1) : 0.0f;
        const float ls1 = lane + 32 < p.splits ? __ldcg(ml + 2 * (lane + 32) + 1) : 0.0f;
        const float m = warp_max(fmaxf(ms0, ms1));
        const float wgt0 = ms0 == -INFINITY ? 0.0f : fast_exp2(ms0 - m);
        const float wgt1 = ms1 == -INFINITY ? 0.0f : fast_exp2(ms1 - m);
        const float l = warp_sum(ls0 * wgt0 + ls1 * wgt1);
        float f = l > 0.0f ? 1.0f / l : 0.0f;
        if (p.gate != nullptr) f *= 1.0f / (1.0f + __expf(-__bfloat162float(p.gate[(int64_t)t * p.ld_gate + h])));
        w_sm[r * 64 + lane] = wgt0;
        w_sm[r * 64 + 32 + lane] = wgt1;
        if (lane == 0) f_sm[r] = f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows_valid * (D / 2); idx += NTHREADS) {
        const int r = idx / (D / 2), d = (idx % (D / 2)) * 2;
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const int64_t row = (int64_t)t * p.Hq + h;
        const float* po = p.part_o + row * p.splits * D + d;
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 8
        for (int s = 0; s < p.splits; ++s) {
            const float w = w_sm[r * 64 + s];
            const float2 raw = __ldcg(reinterpret_cast<const float2*>(po + (int64_t)s * D));
            const float2 v = w == 0.0f ? make_float2(0.0f, 0.0f) : raw;      // an empty part's slot may hold anything
            a0 = fmaf(w, v.x, a0);
            a1 = fmaf(w, v.y, a1);
        }
        const float f = f_sm[r];
        *reinterpret_cast<__nv_bfloat162*>(p.out + row * D + d) = __floats2bfloat162_rn(a0 * f, a1 * f);
    }
    if (threadIdx.x == 0) *counter = 0;          // ready for the next call
}

// The same decode step for head size 64 with the cache's pages brought in by the TMA unit: a page of keys (or values) of
// one kv head is 64 x 64 contiguous bfloat16, one box of a tensor map over the whole cache, written to shared memory
// with the 128-byte swizzle (16-byte chunk c of row r lands at chunk c ^ (r % 8), where ldmatrix then looks for it
// without bank conflicts). A fifth warp's first lane requests pages as stages fall free; the four consumer warps wait on
// a stage's mbarrier, multiply their 16 keys of the block and hand the stage back, so no warp waits for another inside
// the loop, and the 1,024 predicated 16-byte copies a block cost the four warps before are two instructions. Blocks that
// lie wholly before the sequence's newest position are requested before the wait for the kernel that writes that
// position. Rows past the sequence's end and pages that a window has given back come as they are (stale): their scores
// are replaced (never multiplied) by -inf, and their value rows are zeroed in shared memory by the warp that owns them.
// Every mbarrier wait is bounded (tc_common.cuh); a CTA that gives up sets *status and writes nothing useful.
// (KEEP_L1: the same code as a kernel of its own, so that it can carry its own preference for the split of an SM's memory
// between shared memory and L1 cache: see g_attn_tma_carveout)
template <int NST, bool KEEP_L1>
__global__ void __launch_bounds__(160) attention_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_kv, const AttnParams p,
                                                                   int* status) {
    constexpr int D = 64, LD = D + 8, KSTEPS = D / 16, DTILES = D / 8, CHUNKS = D / 8, QROWS = 16;
    constexpr int kPageBytes = BN * D * 2;                                  // 8 KB
    extern __shared__ __align__(1024) unsigned char smem_tma[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_tma + 1023) & ~(uintptr_t)1023);
    unsigned char* k_sm = base;                                              // [NST][64][128 bytes], swizzled
    unsigned char* v_sm = base + NST * kPageBytes;
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(v_sm + NST * kPageBytes);      // [16][LD]
    __shared__ __align__(8) uint64_t bar_full[NST], bar_empty[NST];
    __shared__ float sm_m[4][QROWS], sm_l[4][QROWS];
    __shared__ int pages_sm[64];
    __shared__ int abort_flag;
    __shared__ bool is_last;

    pdl_launch_dependents();
    if (threadIdx.x == 128)       // the producer's lane: the tensor map on its way before the first copy asks for it
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_kv)) : "memory");
    const int seq = blockIdx.y;
    const int kvh = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int tok_begin = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - tok_begin;
    const int t0 = blockIdx.x * p.tokens_per_tile;
    if (t0 >= q_len) return;
    const int nt = min(p.tokens_per_tile, q_len - t0);
    const int kv_len = p.kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;
    const int hi = pos0 + nt;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int b_lo = lo / BN, nb = (hi + BN - 1) / BN - b_lo;
    const int bs = b_lo + (int)((int64_t)nb * split / p.splits);
    const int be = b_lo + (int)((int64_t)nb * (split + 1) / p.splits);
    const int32_t* table = p.page_table + (int64_t)seq * p.P;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.G;
    const int rows_valid = nt * G;          // <= 16
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < NST; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 4);             // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // this CTA's first 64 page numbers in one coalesced read (the page table is part of the step's description: written
    // before the step's first kernel); blocks beyond them, rare, are looked up one by one
    if (threadIdx.x < 64 && bs + (int)threadIdx.x < be) pages_sm[threadIdx.x] = table[bs + threadIdx.x];
    __syncthreads();
    volatile int* abort_p = &abort_flag;
    auto page_of = [&](int b) { return b - bs < 64 ? pages_sm[b - bs] : table[b]; };

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            // the block that holds the sequence's newest position (written by the kernel before this one) and everything
            // after it wait for that kernel; earlier blocks were written by earlier steps
            const int fresh_from = (kv_len - q_len) / BN;
            bool waited = false;
            for (int b = bs, it = 0; b < be; ++b, ++it) {
                const int s = it % NST;
                if (it >= NST && !mbar_wait(smem_u32(&bar_empty[s]), ((it / NST) & 1) ^ 1, abort_p)) break;
                if (!waited && b >= fresh_from) {
                    pdl_wait();
                    waited = true;
                }
                const int page = page_of(b);
                const uint32_t full = smem_u32(&bar_full[s]);
                if (page >= 0) {
                    mbar_expect_tx(full, 2 * kPageBytes);
                    const int y = ((page * 2 + 0) * p.Hkv + kvh) * BN;
                    tma_load_2d(smem_u32(k_sm + s * kPageBytes), &tmap_kv, 0, y, full);
                    tma_load_2d(smem_u32(v_sm + s * kPageBytes), &tmap_kv, 0, y + p.Hkv * BN, full);
                } else {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full) : "memory");   // a page given back: nothing to bring
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers (warps 0..3)
    pdl_wait();
    for (int c = threadIdx.x; c < QROWS * CHUNKS; c += 128) {
        const int r = c / CHUNKS, ch = c % CHUNKS;
        const bool ok = r < rows_valid;
        const int ti = ok ? r / G : 0, g = ok ? r % G : 0;
        const __nv_bfloat16* src = p.q + ((int64_t)(tok_begin + t0 + ti) * p.Hq + kvh * G + g) * D + ch * 8;
        cp_async16(q_sm + r * LD + ch * 8, src, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
        ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], q_sm + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);

    const int r1 = lane >> 2, r2 = r1 + 8;
    const int pos1 = r1 < rows_valid ? pos0 + r1 / G : -1;
    const int pos2 = r2 < rows_valid ? pos0 + r2 / G : -1;
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
    bool bad = false;

    for (int b = bs, it = 0; b < be; ++b, ++it) {
        const int s = it % NST;
        // (the warp decides together: its lanes poll the same barrier but may give up at different polls)
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_full[s]), (it / NST) & 1, abort_p))) {
            bad = true;
            break;
        }
        unsigned char* ks = k_sm + s * kPageBytes;
        unsigned char* vs = v_sm + s * kPageBytes;
        // value rows of this warp's 16 keys that hold no key of this sequence (past its end, or a page given back):
        // zero, so that a weight of exactly 0 times stale bits stays 0
        const int valid = page_of(b) >= 0 ? min(BN, hi - b * BN) : 0;
        if (valid < warp * 16 + 16) {
            for (int i = lane; i < 16 * CHUNKS; i += 32) {
                const int r = warp * 16 + i / CHUNKS;
                if (r >= valid) *reinterpret_cast<uint4*>(vs + r * 128 + (i % CHUNKS) * 16) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // before the TMA unit writes this stage again
            __syncwarp();
        }
        float sc[2][4];
        sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            unsigned b0, b1, b2, b3;
            const int r = warp * 16 + (lane >> 4) * 8 + (lane & 7), ch = kk * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b0, b1, b2, b3, ks + r * 128 + ((ch ^ (r & 7)) << 4));
            mma_bf16(sc[0], qf[kk], b0, b1);
            mma_bf16(sc[1], qf[kk], b2, b3);
        }
        const int key0 = b * BN + warp * 16 + (lane & 3) * 2;
        float mx1 = -INFINITY, mx2 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + i * 8 + e;
                const bool v1 = key <= pos1 && (p.window == 0 || pos1 - key < p.window);
                const bool v2 = key <= pos2 && (p.window == 0 || pos2 - key < p.window);
                sc[i][e] = v1 ? sc[i][e] * p.scale_log2 : -INFINITY;
                sc[i][2 + e] = v2 ? sc[i][2 + e] * p.scale_log2 : -INFINITY;
                mx1 = fmaxf(mx1, sc[i][e]);
                mx2 = fmaxf(mx2, sc[i][2 + e]);
            }
        }
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 1));
        mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 2));
        const float mn1 = fmaxf(m1, mx1), mn2 = fmaxf(m2, mx2);
        const float base1 = mn1 == -INFINITY ? 0.0f : mn1, base2 = mn2 == -INFINITY ? 0.0f : mn2;
        const float c1 = fast_exp2(m1 - base1), c2 = fast_exp2(m2 - base2);
        m1 = mn1;
        m2 = mn2;
        l1 *= c1;
        l2 *= c2;
#pragma unroll
        for (int i = 0; i < DTILES; ++i) {
            o[i][0] *= c1;
            o[i][1] *= c1;
            o[i][2] *= c2;
            o[i][3] *= c2;
        }
        unsigned pf[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float p0 = fast_exp2(sc[i][0] - base1), p1 = fast_exp2(sc[i][1] - base1);
            const float p2 = fast_exp2(sc[i][2] - base2), p3 = fast_exp2(sc[i][3] - base2);
            l1 += p0 + p1;
            l2 += p2 + p3;
            pf[i * 2 + 0] = pack_bf16(p0, p1);
            pf[i * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            unsigned b0, b1, b2, b3;
            const int r = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), ch = dp * 2 + (lane >> 4);
            ldmatrix_x4_trans(b0, b1, b2, b3, vs + r * 128 + ((ch ^ (r & 7)) << 4));
            mma_bf16(o[2 * dp], pf, b0, b1);
            mma_bf16(o[2 * dp + 1], pf, b2, b3);
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_empty[s])) : "memory");
    }
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    l2 += __shfl_xor_sync(0xffffffffu, l2, 1);
    l2 += __shfl_xor_sync(0xffffffffu, l2, 2);

    // ---- merge the four warps through the (now idle) key stages: every consumer comes here, whatever happened before
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*abort_p || bad) {
        if (threadIdx.x == 0) atomicExch(status, 1);
        return;                              // (the same for all 128: the flag was set before the barrier, or never)
    }
    float* sm_o = reinterpret_cast<float*>(k_sm);          // [4][16][D] = 16 KB: two stages' keys
    if ((lane & 3) == 0) {
        sm_m[warp][r1] = m1;
        sm_l[warp][r1] = l1;
        sm_m[warp][r2] = m2;
        sm_l[warp][r2] = l2;
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
        float* d1 = sm_o + ((warp * QROWS + r1) * D) + i * 8 + (lane & 3) * 2;
        float* d2 = sm_o + ((warp * QROWS + r2) * D) + i * 8 + (lane & 3) * 2;
        d1[0] = o[i][0];
        d1[1] = o[i][1];
        d2[0] = o[i][2];
        d2[1] = o[i][3];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    for (int idx = threadIdx.x; idx < rows_valid * D; idx += 128) {
        const int r = idx / D, d = idx % D;
        float m = fmaxf(fmaxf(sm_m[0][r], sm_m[1][r]), fmaxf(sm_m[2][r], sm_m[3][r]));
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = sm_m[w][r] == -INFINITY ? 0.0f : fast_exp2(sm_m[w][r] - m);
            l += sm_l[w][r] * f;
            acc += sm_o[(w * QROWS + r) * D + d] * f;
        }
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const int64_t row = (int64_t)t * p.Hq + h;
        if (p.splits == 1) {
            float f = l > 0.0f ? 1.0f / l : 0.0f;
            if (p.gate != nullptr) f *= 1.0f / (1.0f + __expf(-__bfloat162float(p.gate[(int64_t)t * p.ld_gate + h])));
            p.out[row * D + d] = __float2bfloat16_rn(acc * f);
        } else {
            p.part_o[(row * p.splits + split) * D + d] = acc;
            if (d == 0) {
                p.part_ml[(row * p.splits + split) * 2 + 0] = m;
                p.part_ml[(row * p.splits + split) * 2 + 1] = l;
            }
        }
    }
    if (p.splits == 1 || p.counters == nullptr) return;
    // ---- the CTA of a (sequence, kv head) that stores its part last merges all of them (as attention_decode_mma_kernel)
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    unsigned int* counter = p.counters + (int64_t)seq * p.Hkv + kvh;
    if (threadIdx.x == 0) is_last = atomicAdd(counter, 1u) == (unsigned)p.splits - 1;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!is_last) return;
    __threadfence();
    float* w_sm = reinterpret_cast<float*>(v_sm);            // [rows][64] weights, then [rows] 1 / sum (times the gate)
    float* f_sm = w_sm + QROWS * 64;
    for (int r = warp; r < rows_valid; r += 4) {
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const float* ml = p.part_ml + ((int64_t)t * p.Hq + h) * p.splits * 2;
        const float ms0 = lane < p.splits ? __ldcg(ml + 2 * lane) : -INFINITY;
        const float ms1 = lane + 32 < p.splits ? __ldcg(ml + 2 * (lane + 32)) : -INFINITY;
        const float ls0 = lane < p.splits ? __ldcg(ml + 2 * lane + 1) : 0.0f;
        const float ls1 = lane + 32 < p.splits ? __ldcg(ml + 2 * (lane + 32) + 1) : 0.0f;
        const float m = warp_max(fmaxf(ms0, ms1));
        const float wgt0 = ms0 == -INFINITY ? 0.0f : fast_exp2(ms0 - m);
        const float wgt1 = ms1 == -INFINITY ? 0.0f : fast_exp2(ms1 - m);
        const float l = warp_sum(ls0 * wgt0 + ls1 * wgt1);
        float f = l > 0.0f ? 1.0f / l : 0.0f;
        if (p.gate != nullptr) f *= 1.0f / (1.0f + __expf(-__bfloat162float(p.gate[(int64_t)t * p.ld_gate + h])));
        w_sm[r * 64 + lane] = wgt0;
        w_sm[r * 64 + 32 + lane] = wgt1;
        if (lane == 0) f_sm[r] = f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    for (int idx = threadIdx.x; idx < rows_valid * (D / 2); idx += 128) {
        const int r = idx / (D / 2), d = (idx % (D / 2)) * 2;
        const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
        const int64_t row = (int64_t)t * p.Hq + h;
        const float* po = p.part_o + row * p.splits * D + d;
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 8
        for (int s = 0; s < p.splits; ++s) {
            const float w = w_sm[r * 64 + s];
            const float2 raw = __ldcg(reinterpret_cast<const float2*>(po + (int64_t)s * D));
            const float2 v = w == 0.0f ? make_float2(0.0f, 0.0f) : raw;
            a0 = fmaf(w, v.x, a0);
            a1 = fmaf(w, v.y, a1);
        }
        const float f = f_sm[r];
        *reinterpret_cast<__nv_bfloat162*>(p.out + row * D + d) = __floats2bfloat162_rn(a0 * f, a1 * f);
    }
    if (threadIdx.x == 0) *counter = 0;
}

// out[row, :] = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), times the head's gate. One warp per row; lane s holds
// splits s and s + 32's (max, sum) and weights (splits <= 64), and the partial outputs are read with independent loads.
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const __nv_bfloat16* __restrict__ gate, int64_t ld_gate,
                                         __nv_bfloat16* __restrict__ out, int64_t rows, int Hq, int D, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* ml = part_ml + row * splits * 2;
    // lane s holds splits s and s + 32
    const float ms0 = lane < splits ? ml[2 * lane] : -INFINITY, ms1 = lane + 32 < splits ? ml[2 * (lane + 32)] : -INFINITY;
    const float ls0 = lane < splits ? ml[2 * lane + 1] : 0.0f, ls1 = lane + 32 < splits ? ml[2 * (lane + 32) + 1] : 0.0f;
    const float m = warp_max(fmaxf(ms0, ms1));
    const float wgt0 = ms0 == -INFINITY ? 0.0f : fast_exp2(ms0 - m);     // the splits' weights
    const float wgt1 = ms1 == -INFINITY ? 0.0f : fast_exp2(ms1 - m);
    const float l = warp_sum(ls0 * wgt0 + ls1 * wgt1);
    float f = l > 0.0f ? 1.0f / l : 0.0f;
    if (gate != nullptr) {
        const int64_t t = row / Hq;
        const int h = (int)(row % Hq);
        f *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[t * ld_gate + h])));
    }
    const float* po = part_o + row * splits * D;
    for (int d0 = 0; d0 < D; d0 += 64) {       // every lane stays in the loop: the shuffles need the whole warp
        const int d = d0 + 2 * lane;           // D is a multiple of 16: a lane's two channels are both inside or both outside
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 16
        for (int s = 0; s < splits; ++s) {
            const float w = __shfl_sync(0xffffffffu, s < 32 ? wgt0 : wgt1, s & 31);
            // (read whatever the weight: the loads then wait for nothing but the row's address; an empty part's
            // slot may hold anything, so its value is dropped, not multiplied by zero)
            const float2 raw = d < D ? *reinterpret_cast<const float2*>(po + s * D + d) : make_float2(0.0f, 0.0f);
            const float2 v = w == 0.0f ? make_float2(0.0f, 0.0f) : raw;
            a0 = fmaf(w, v.x, a0);
            a1 = fmaf(w, v.y, a1);
        }
        if (d < D) *reinterpret_cast<__nv_bfloat162*>(out + row * D + d) = __floats2bfloat162_rn(a0 * f, a1 * f);
    }
}

template <int D, int NST>
int launch_stages(const AttnParams& p, int max_tiles, int n_seqs, cudaStream_t stream) {
    constexpr int LD = D + 8;
    const size_t smem = (size_t)(BM + 2 * NST * BN) * LD * sizeof(__nv_bfloat16);
    static bool opted = false;
    if (smem > 48 * 1024 && !opted) {
        cudaFuncSetAttribute(attention_mma_kernel<D, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        opted = true;
    }
    const dim3 grid(max_tiles, n_seqs, p.Hkv * p.splits);
    xs_launch(attention_mma_kernel<D, NST>, grid, dim3(NTHREADS), smem, stream, p);
    return 0;
}

// Prompts (many query tiles, compute-bound): two stages. Decoding (one tile a sequence, bound by the latency of the
// cache reads): four stages, so that three 64-key blocks are on their way while one is used.
int g_attn_decode_stages = 4;
int g_attn_prefetch_blocks = 2;

template <int D, int NST>
int launch_decode(const AttnParams& p, int n_seqs, cudaStream_t stream) {
    constexpr int LD = D + 8;
    const size_t smem = (size_t)(16 + 2 * NST * BN) * LD * sizeof(__nv_bfloat16);
    static bool opted = false;
    if (smem > 48 * 1024 && !opted) {
        cudaFuncSetAttribute(attention_decode_mma_kernel<D, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        opted = true;
    }
    const dim3 grid(1, n_seqs, p.Hkv * p.splits);
    xs_launch(attention_decode_mma_kernel<D, NST>, grid, dim3(NTHREADS), smem, stream, p);
    return 0;
}

// Decoding at head size 64 through the TMA-fed kernel: `map` covers the whole cache as rows of 64 elements.
int g_attn_decode_tma = 1;        // 0: the cp.async kernel for every head size (xs_attention_mma_set_decode_tma)
int g_attn_tma_stages = 3;
// Shared-memory carveout (per cent of an SM's 228 KB) that the TMA-fed kernel asks for while sequences x kv heads (its CTAs
// before any key split) are at most three an SM: 164 KB hold three CTAs, and 64 KB stay L1 cache. Measured on B200 (1.2B shape, batch 8, whole decode step): with the
// driver's own choice for four CTAs an SM (the whole 228 KB) the step takes 0.89 ms instead of 0.75: the few-row products
// before and after overlap this kernel on its SMs and then read their activations without an L1. Larger grids (batch 64:
// 1.16 ms against 1.27) want the fourth CTA more. 0: always the driver's choice.
int g_attn_tma_carveout = 72;

int sm_count();

template <int NST, bool KEEP_L1>
int launch_decode_tma_as(const AttnParams& p, const CUtensorMap& map, int* status, int n_seqs, cudaStream_t stream) {
    const size_t smem = (size_t)2 * NST * BN * 64 * sizeof(__nv_bfloat16) + (size_t)16 * 72 * sizeof(__nv_bfloat16) + 1024;
    static bool opted = false;
    if (!opted) {
        cudaFuncSetAttribute(attention_decode_tma_kernel<NST, KEEP_L1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (KEEP_L1)
            cudaFuncSetAttribute(attention_decode_tma_kernel<NST, KEEP_L1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 g_attn_tma_carveout);
        opted = true;
    }
    const dim3 grid(1, n_seqs, p.Hkv * p.splits);
    xs_launch(attention_decode_tma_kernel<NST, KEEP_L1>, grid, dim3(160), smem, stream, map, p, status);
    return 0;
}

// Few CTAs before any key split (sequences x kv heads at most three an SM): the instance that keeps an L1.
bool tma_keeps_l1(int64_t tiles) { return g_attn_tma_carveout > 0 && tiles <= (int64_t)3 * sm_count(); }

template <int NST>
int launch_decode_tma(const AttnParams& p, const CUtensorMap& map, int* status, int n_seqs, cudaStream_t stream) {
    if (tma_keeps_l1((int64_t)n_seqs * p.Hkv)) return launch_decode_tma_as<NST, true>(p, map, status, n_seqs, stream);
    return launch_decode_tma_as<NST, false>(p, map, status, n_seqs, stream);
}

template <int D, int NST>
int decode_ctas_per_sm() {
    static int cached[16] = {};                  // per device: the answer does not change
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && cached[dev] > 0) return cached[dev];
    constexpr int LD = D + 8;
    const size_t smem = (size_t)(16 + 2 * NST * BN) * LD * sizeof(__nv_bfloat16);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(attention_decode_mma_kernel<D, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_mma_kernel<D, NST>, NTHREADS, smem) != cudaSuccess)
        n = 0;
    if (dev >= 0 && dev < 16) cached[dev] = n;
    return n;
}

int sm_count() {
    static int cached[16] = {};
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && cached[dev] > 0) return cached[dev];
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (dev >= 0 && dev < 16) cached[dev] = n;
    return n;
}

// Stages of the decode kernel for `tiles` (sequences x kv heads) CTAs before any key split. Three stages keep more
// of a CTA's keys in flight and win while the CTAs of one round fit the device (measured on B200, 8 sequences of
// 2,048 keys: 13.5 against 14.6 us). When even one CTA a tile is more than the three-stage kernel places at one
// time, two stages let five CTAs share an SM instead of three (64 sequences of 2,048 keys: 52.9 against 62.7 us).
template <int D>
int decode_stages_for(int64_t tiles) {
    if (g_attn_decode_stages <= 3) return g_attn_decode_stages < 3 ? 2 : 3;      // asked for by the caller
    return tiles > (int64_t)sm_count() * decode_ctas_per_sm<D, 3>() ? 2 : 3;
}

template <int D>
int launch(const AttnParams& p, int max_tiles, int n_seqs, cudaStream_t stream) {
    if (p.decode_rows && decode_stages_for<D>((int64_t)n_seqs * p.Hkv) >= 3) return launch_decode<D, 3>(p, n_seqs, stream);
    if (p.decode_rows) return launch_decode<D, 2>(p, n_seqs, stream);
    if (max_tiles == 1 && D <= 64 && g_attn_decode_stages >= 4) return launch_stages<D, 4>(p, max_tiles, n_seqs, stream);
    if (max_tiles == 1 && g_attn_decode_stages >= 3) return launch_stages<D, 3>(p, max_tiles, n_seqs, stream);
    return launch_stages<D, 2>(p, max_tiles, n_seqs, stream);
}

}  // namespace

// How many of its first key blocks a decode CTA hints into L2 before it waits for the previous kernel; returns the
// previous value.
XS_API int xs_attention_mma_set_prefetch_blocks(int n) {
    const int old = g_attn_prefetch_blocks;
    g_attn_prefetch_blocks = n;
    return old;
}

// How many cp.async stages decoding uses: 2 or 3 as given, 4 (the default) chooses by the number of tiles; returns
// the previous value.
XS_API int xs_attention_mma_set_decode_stages(int n) {
    const int old = g_attn_decode_stages;
    g_attn_decode_stages = n;
    return old;
}

// CTAs of the decode kernel (one token a sequence) that run at one time on this device when `tiles` = sequences x kv
// heads (the number of stages, and with it the CTAs an SM, follows from that); 0 when the head size is not
// supported. The caller sizes its key splits by it.
namespace {
template <int D>
int decode_slots(int64_t tiles) {
    return sm_count() * (decode_stages_for<D>(tiles) >= 3 ? decode_ctas_per_sm<D, 3>() : decode_ctas_per_sm<D, 2>());
}
}  // namespace
XS_API int xs_attention_mma_decode_slots(int D, int64_t tiles) {
    if (D == 64 && g_attn_decode_tma && encode_fn() != nullptr) {       // the TMA-fed kernel: its own occupancy
        static int per_sm[8][2] = {};
        const int n = g_attn_tma_stages, k = tma_keeps_l1(tiles) ? 1 : 0;
        if (per_sm[n][k] == 0) {
            const size_t smem = (size_t)2 * n * BN * 64 * sizeof(__nv_bfloat16) + (size_t)16 * 72 * sizeof(__nv_bfloat16) + 1024;
            int got = 0;
#define XS_TMA_OCC(NST, KEEP)                                                                                                \
    do {                                                                                                                     \
        cudaFuncSetAttribute(attention_decode_tma_kernel<NST, KEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (KEEP)                                                                                                            \
            cudaFuncSetAttribute(attention_decode_tma_kernel<NST, KEEP>, cudaFuncAttributePreferredSharedMemoryCarveout,     \
                                 g_attn_tma_carveout);                                                                       \
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&got, attention_decode_tma_kernel<NST, KEEP>, 160, smem);              \
    } while (0)
#define XS_TMA_OCC2(NST) if (k) XS_TMA_OCC(NST, true); else XS_TMA_OCC(NST, false)
            switch (n) {
                case 2: XS_TMA_OCC2(2); break;
                case 3: XS_TMA_OCC2(3); break;
                case 5: XS_TMA_OCC2(5); break;
                case 6: XS_TMA_OCC2(6); break;
                default: XS_TMA_OCC2(4); break;
            }
#undef XS_TMA_OCC2
#undef XS_TMA_OCC
            // (the occupancy query may not know of the carveout: 164 KB hold three CTAs of three stages)
            if (k && got > (int)((size_t)g_attn_tma_carveout * 228 * 1024 / 100 / (smem + 1024))) got = (int)((size_t)g_attn_tma_carveout * 228 * 1024 / 100 / (smem + 1024));
            per_sm[n][k] = got > 0 ? got : 1;
        }
        return sm_count() * per_sm[n][k];
    }
    switch (D) {
        case 16: return decode_slots<16>(tiles);
        case 32: return decode_slots<32>(tiles);
        case 48: return decode_slots<48>(tiles);
        case 64: return decode_slots<64>(tiles);
        case 96: return decode_slots<96>(tiles);
        case 128: return decode_slots<128>(tiles);
        default: return 0;
    }
}

// Scratch the split path needs, in bytes, for `rows` = tokens * heads.
XS_API int64_t xs_attention_mma_scratch_bytes(int64_t rows, int D, int splits) {
    return splits <= 1 ? 0 : rows * splits * ((int64_t)D + 2) * (int64_t)sizeof(float);
}

// 1 when xs_attention_mma takes this head size and page size.
XS_API int xs_attention_mma_supports(int D, int page_size, int G) {
    const bool d_ok = D == 16 || D == 32 || D == 48 || D == 64 || D == 96 || D == 128;
    return d_ok && page_size == BN && G >= 1 && G <= BM;
}

XS_API void xs_attention_mma_set_decode_tma(int on, int stages) {
    g_attn_decode_tma = on ? 1 : 0;
    if (stages >= 2 && stages <= 6) g_attn_tma_stages = stages;
}
XS_API void xs_attention_mma_set_tma_carveout(int percent) { g_attn_tma_carveout = percent; }

// `counters` (or null): n_seqs * Hkv zeroed words, left zeroed. With them, when every sequence brings one token and its
// keys are split, the CTA of a (sequence, kv head) that finishes last merges the parts, and no second kernel is launched.
// `status` (or null) with `pool_pages` (the cache's first dimension): one device int that a kernel with bounded waits sets
// non-zero when a wait gave up (the result is then invalid); with them, decoding at head size 64 takes the TMA-fed kernel.
XS_API int xs_attention_mma_merged(const void* q, const void* pool, const int32_t* page_table, int P,
                                   const int32_t* cu_seqlens, const int32_t* kv_lens, const void* gate, int64_t ld_gate,
                                   void* out, void* scratch, int64_t scratch_bytes, void* counters, int64_t pool_pages,
                                   int* status, int T, int n_seqs, int max_q_len, int Hq, int Hkv, int D, int page_size,
                                   float scale, int window, int splits, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: %d heads over %d kv heads", Hq, Hkv);
    const int G = Hq / Hkv;
    XS_REQUIRE(xs_attention_mma_supports(D, page_size, G),
               "attention (tensor cores): head size %d, page size %d, group %d is not supported", D, page_size, G);
    XS_REQUIRE(splits >= 1 && splits <= 64 && window >= 0 && max_q_len >= 1 && n_seqs >= 1 && P >= 1,
               "attention: bad sizes (1 to 64 key splits)");
    XS_REQUIRE(n_seqs <= 65535 && (int64_t)Hkv * splits <= 65535, "attention: grid too large");
    const int64_t need = xs_attention_mma_scratch_bytes((int64_t)T * Hq, D, splits);
    XS_REQUIRE((uintptr_t)out % 4 == 0 && (splits == 1 || (uintptr_t)scratch % 16 == 0), "attention: out or scratch is misaligned");
    XS_REQUIRE(splits == 1 || (scratch != nullptr && scratch_bytes >= need),
               "attention: %lld bytes of scratch needed for %d splits, %lld given", (long long)need, splits,
               (long long)scratch_bytes);
    AttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.pool = (const __nv_bfloat16*)pool;
    p.page_table = page_table;
    p.P = P;
    p.cu_seqlens = cu_seqlens;
    p.kv_lens = kv_lens;
    p.gate = (const __nv_bfloat16*)gate;
    p.ld_gate = ld_gate;
    p.out = (__nv_bfloat16*)out;
    p.part_o = (float*)scratch;
    p.part_ml = p.part_o + (int64_t)T * Hq * splits * D;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = G;
    p.tokens_per_tile = BM / G;
    p.decode_rows = (max_q_len == 1 && G <= 16) ? 1 : 0;
    p.window = window;
    p.splits = splits;
    p.prefetch_blocks = g_attn_prefetch_blocks;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.counters = (p.decode_rows && splits > 1) ? (unsigned int*)counters : nullptr;
    const int max_tiles = ceil_div_i(max_q_len, p.tokens_per_tile);
    if (p.decode_rows && D == 64 && g_attn_decode_tma && status != nullptr && pool_pages > 0 && (uintptr_t)pool % 16 == 0 &&
        encode_fn() != nullptr) {
        alignas(64) CUtensorMap map;
        XS_REQUIRE(make_map(&map, pool, pool_pages * 2 * Hkv * BN, D, D, BN), "attention: the cache's tensor map could not be made");
        switch (g_attn_tma_stages) {
            case 2: launch_decode_tma<2>(p, map, status, n_seqs, stream); break;
            case 3: launch_decode_tma<3>(p, map, status, n_seqs, stream); break;
            case 5: launch_decode_tma<5>(p, map, status, n_seqs, stream); break;
            case 6: launch_decode_tma<6>(p, map, status, n_seqs, stream); break;
            default: launch_decode_tma<4>(p, map, status, n_seqs, stream); break;
        }
    } else
    switch (D) {
        case 16: launch<16>(p, max_tiles, n_seqs, stream); break;
        case 32: launch<32>(p, max_tiles, n_seqs, stream); break;
        case 48: launch<48>(p, max_tiles, n_seqs, stream); break;
        case 64: launch<64>(p, max_tiles, n_seqs, stream); break;
        case 96: launch<96>(p, max_tiles, n_seqs, stream); break;
        case 128: launch<128>(p, max_tiles, n_seqs, stream); break;
        default: XS_REQUIRE(false, "attention (tensor cores): head size %d", D);
    }
    XS_LAUNCH_CHECK("attention_mma");
    if (splits > 1 && p.counters == nullptr) {
        const int64_t rows = (int64_t)T * Hq;
        xs_launch(attention_combine_kernel, dim3(ceil_div_i(rows, 4)), dim3(128), 0, stream, (const float*)p.part_o,
                  (const float*)p.part_ml, p.gate, ld_gate, p.out, rows, Hq, D, splits);
        XS_LAUNCH_CHECK("attention_combine");
    }
    return 0;
}

XS_API int xs_attention_mma(const void* q, const void* pool, const int32_t* page_table, int P,
                            const int32_t* cu_seqlens, const int32_t* kv_lens, const void* gate, int64_t ld_gate,
                            void* out, void* scratch, int64_t scratch_bytes, int T, int n_seqs, int max_q_len, int Hq,
                            int Hkv, int D, int page_size, float scale, int window, int splits, cudaStream_t stream) {
    return xs_attention_mma_merged(q, pool, page_table, P, cu_seqlens, kv_lens, gate, ld_gate, out, scratch, scratch_bytes,
                                   nullptr, 0, nullptr, T, n_seqs, max_q_len, Hq, Hkv, D, page_size, scale, window, splits,
                                   stream);
}

// ------------------------------------------------------------------------------------------------
// The same operation for callers that cannot allocate (xs_no_alloc.h): the scratch for the partial
// results is a device array that is part of the library image.
#include "xs_no_alloc.h"

namespace {
constexpr int64_t kScratchBytes = 8ll * 1024 * 1024;
constexpr int kMaxDevices = 64;
// In host code this name is only a handle for the runtime, not a device address; the address that
// kernels may use comes from cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];
void* g_static_scratch_ptr[kMaxDevices] = {};
}  // namespace

XS_API int64_t xs_attention_mma_static_capacity(void) { return kScratchBytes; }

XS_API int xs_attention_mma_static(const void* q, const void* pool, const int32_t* page_table, int P,
                                   const int32_t* cu_seqlens, const int32_t* kv_lens, const void* gate,
                                   int64_t ld_gate, void* out, int T, int n_seqs, int max_q_len, int Hq, int Hkv,
                                   int D, int page_size, float scale, int window, int splits, cudaStream_t stream) {
    XS_REQUIRE(T >= 0 && Hq > 0 && D > 0 && splits >= 1, "attention (built-in scratch): bad sizes");
    const int64_t need = xs_attention_mma_scratch_bytes((int64_t)T * Hq, D, splits);
    XS_REQUIRE(need <= kScratchBytes,
               "attention (built-in scratch): %d tokens x %d heads x %d splits need %lld bytes of scratch, the "
               "built-in array holds %lld; use fewer splits or xs_attention_mma with a buffer of your own",
               T, Hq, splits, (long long)need, (long long)kScratchBytes);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    XS_REQUIRE(e == cudaSuccess && device >= 0 && device < kMaxDevices, "attention (built-in scratch): no usable current device (%s)",
               cudaGetErrorString(e));
    if (g_static_scratch_ptr[device] == nullptr) {   // first call on this device: not inside a stream capture
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        XS_REQUIRE(e == cudaSuccess && ptr != nullptr, "attention (built-in scratch): cudaGetSymbolAddress failed: %s",
                   cudaGetErrorString(e));
        g_static_scratch_ptr[device] = ptr;
    }
    return xs_attention_mma(q, pool, page_table, P, cu_seqlens, kv_lens, gate, ld_gate, out, g_static_scratch_ptr[device],
                            kScratchBytes, T, n_seqs, max_q_len, Hq, Hkv, D, page_size, scale, window, splits, stream);
}
