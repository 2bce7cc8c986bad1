// Prefill attention over the paged bfloat16 cache on Blackwell's fifth-generation tensor cores.
//
// One CTA owns a tile of 128 query rows that share one kv head (row r = token r / G, head r % G of the
// group, G = heads / kv_heads) and walks the cache in blocks of 128 keys (two pages). Per block:
//
//   warp 0   TMA producer: the block's K and V pages (64 x 64 elements each, 128-byte swizzle) into a
//            ring of three stages. Pages past the sequence's end, pages a window has given back, and the
//            rows of the last page past the sequence's length are zeroed in shared memory (V only: a
//            masked score becomes a weight of exactly 0, and 0 times stale bits must stay 0).
//   warp 1 and warp 10: one thread each issues S = Q K^T and O += P V:
//   warp 1   one thread issues S = Q K^T (tcgen05.mma, M 128, N 128, K 16 x D / 16, Q and K K-major) into
//            one of two S buffers in tensor memory, and O += P V (M 128, N D, K 16 x 8, P K-major from
//            shared memory, V MN-major: the pages' own layout) into the output, which stays in tensor memory.
//   warps 2-9 softmax, two threads a query row (64 keys of the block each): tcgen05.ld of S, mask (causal,
//            window), running maximum and sum in float32 with base-2 exponentials, P as bfloat16 into
//            shared memory (swizzled by hand as TMA would have). When a row's maximum moves, its threads
//            rescale their halves of its output in tensor memory (tcgen05.ld, multiply, tcgen05.st) before
//            they hand the block's P over; the output is read once, at the end.
//
// S of block j + 1 is issued before P V of block j, so the tensor pipe works while the softmax of block j
// runs. Every mbarrier wait is bounded (see tc_common.cuh); a CTA that gives up frees its tensor memory and
// sets *status. Head size 64, groups that divide 128, one key split; other cases take the mma.sync kernel.
// The reference's counterpart is its XMX flash kernel for prefill (src/backend/sycl/sycl_flash_attention.cpp:1-15).
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int TM = 128;           // query rows a CTA
constexpr int TN = 128;           // keys a block
constexpr int PAGE = 64;          // keys a page
constexpr int kAttnThreads = 352;   // TMA warp, S issuer warp, eight softmax warps, P V issuer warp
constexpr int KV_STAGES = 3;

struct AttnTcParams {
    const __nv_bfloat16* q;          // [T, Hq, D]
    const int32_t* page_table;       // [n_seqs, P]
    int P;
    const int32_t* cu_seqlens;
    const int32_t* kv_lens;
    const __nv_bfloat16* gate;       // [T, ld_gate] or null
    int64_t ld_gate;
    __nv_bfloat16* out;              // [T, Hq, D]
    int* status;
    int Hq, Hkv, G, tokens_per_tile, window;
    float scale_log2;
    int order;
};

__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Writes of this thread to shared memory become visible to the tensor core's and the TMA unit's reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// tcgen05.ld of 32 columns without waiting for them: several can be in flight before one tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t addr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16w(uint32_t addr, uint32_t* r) {     // 16 columns, waited for
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16w(uint32_t addr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 :: "r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                    "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// tcgen05.st of 32 columns of this thread's lane, and the wait for it
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        :: "r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
           "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
           "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
           "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Descriptor of an MN-major operand with the 128-byte swizzle: 64 elements of N contiguous (128 bytes), rows of
// K 128 bytes apart, groups of 8 rows of K 1024 bytes apart (stride byte offset). One 64-wide chunk of N only,
// so the leading byte offset is not used.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_kv, const AttnTcParams p) {
    static_assert(D == 64, "one 128-byte swizzle atom a row");
    constexpr int kPageBytes = PAGE * D * 2;                   // 8 KB
    constexpr int kStageBytes = 4 * kPageBytes;                // K (two pages), V (two pages)
    constexpr int kPBytes = TM * TN * 2;                       // 32 KB: two halves of 64 keys
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_sm = base;
    uint8_t* kv_sm = q_sm + TM * D * 2;
    uint8_t* p_sm = kv_sm + KV_STAGES * kStageBytes;
    __shared__ __align__(8) uint64_t bar_kv_full[KV_STAGES], bar_kv_empty[KV_STAGES], bar_fix[KV_STAGES];
    __shared__ __align__(8) uint64_t bar_s_full[2], bar_s_empty[2], bar_p_full[2], bar_o_done[2];
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;

    pdl_launch_dependents();
    pdl_wait();
    // later tiles see more keys: they are started first, so that the short ones fill the tail; with p.order those of
    // all kv heads before any earlier tile (the grid is (tiles, sequences, kv heads); CTAs start in the order of their
    // flat index)
    int tile, seq, kvh;
    if (p.order) {
        const int flat = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        kvh = flat % (int)gridDim.z;
        seq = (flat / (int)gridDim.z) % (int)gridDim.y;
        tile = (int)gridDim.x - 1 - flat / (int)(gridDim.z * gridDim.y);
    } else {
        tile = gridDim.x - 1 - blockIdx.x, seq = blockIdx.y, kvh = blockIdx.z;
    }
    const int tok_begin = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - tok_begin;
    const int t0 = tile * p.tokens_per_tile;
    if (t0 >= q_len) return;                                   // the whole CTA, before anything is set up
    const int nt = min(p.tokens_per_tile, q_len - t0);
    const int kv_len = p.kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;
    const int hi = pos0 + nt;                                  // keys [lo, hi) matter to this tile
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int b_lo = lo / TN, nb = (hi + TN - 1) / TN - b_lo;
    const int32_t* table = p.page_table + (int64_t)seq * p.P;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.G;
    const int rows_valid = nt * G;
    constexpr uint32_t kTmemCols = 512;                        // S0, S1 (128 each), O (D): 320 of the 512 are used
    constexpr uint32_t kColO = 2 * TN;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(smem_u32(&bar_kv_full[s]), 1);
            mbar_init(smem_u32(&bar_kv_empty[s]), 1);
            mbar_init(smem_u32(&bar_fix[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_o_done[b]), 1);
            mbar_init(smem_u32(&bar_s_full[b]), 1);
            mbar_init(smem_u32(&bar_s_empty[b]), 4);           // one arrival per softmax warp of the buffer's group
            mbar_init(smem_u32(&bar_p_full[b]), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 2 && warp < 6) {
        // ---- Q tile: row r = (token t0 + r / G, head kvh * G + r % G), zero beyond the tile's rows; chunk c of a
        // row sits at chunk c ^ (r % 8), which is where the 128-byte swizzle looks for it
        const int r = (warp & 3) * 32 + lane;
        const bool ok = r < rows_valid;
        const __nv_bfloat16* src = p.q + ((int64_t)(tok_begin + t0 + (ok ? r / G : 0)) * p.Hq + kvh * G + (ok ? r % G : 0)) * D;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            const uint4 v = ok ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(q_sm + r * 128 + ((c ^ (r & 7)) << 4)) = v;
        }
        fence_async_smem();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    volatile int* abort_p = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        int fixes[KV_STAGES];
#pragma unroll
        for (int s = 0; s < KV_STAGES; ++s) fixes[s] = 0;
        for (int j = 0; j < nb && !*abort_p; ++j) {
            const int s = j % KV_STAGES;
            // (the warp decides together: its lanes poll the same barrier but may give up at different polls)
            if (j >= KV_STAGES && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_kv_empty[s]), ((j / KV_STAGES) & 1) ^ 1, abort_p))) break;
            uint8_t* stage = kv_sm + s * kStageBytes;
            int page[2], valid[2];                             // physical page (-1: none), rows of it inside the sequence
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int lp = 2 * (b_lo + j) + h;
                const int rows = min(PAGE, kv_len - lp * PAGE);
                page[h] = (rows > 0 && lp < p.P) ? table[lp] : -1;
                valid[h] = page[h] >= 0 ? rows : 0;
            }
            const bool fix = valid[0] < PAGE || valid[1] < PAGE;
            const uint32_t bytes = (uint32_t)((page[0] >= 0) + (page[1] >= 0)) * 2u * kPageBytes;
            const uint32_t bar = smem_u32(fix ? &bar_fix[s] : &bar_kv_full[s]);
            if (lane == 0) {
                if (bytes > 0) mbar_expect_tx(bar, bytes); else mbar_arrive_cta(bar);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (page[h] < 0) continue;
                    const int y = ((page[h] * 2 + 0) * p.Hkv + kvh) * PAGE;
                    tma_load_2d(smem_u32(stage + h * kPageBytes), &tmap_kv, 0, y, bar);
                    tma_load_2d(smem_u32(stage + 2 * kPageBytes + h * kPageBytes), &tmap_kv, 0, y + p.Hkv * PAGE, bar);
                }
            }
            if (fix) {
                // wait for what was loaded, zero V's rows that hold no key of this sequence, hand the stage over
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_fix[s]), fixes[s] & 1, abort_p))) break;
                ++fixes[s];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint8_t* v_page = stage + 2 * kPageBytes + h * kPageBytes;
                    for (int i = valid[h] * 8 + lane; i < PAGE * 8; i += 32)      // 16-byte chunks from row valid[h] on
                        *reinterpret_cast<uint4*>(v_page + i * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cta(smem_u32(&bar_kv_full[s]));
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ issuer of S = Q K^T
        // (two issuing threads, this one and warp 10's: one thread's descriptor arithmetic and waits for both
        // products of a block took longer than the block's softmax)
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc_mn(TM, TN);
            const uint64_t dq = smem_desc_sw128(smem_u32(q_sm));
            const uint64_t dk0 = smem_desc_sw128(smem_u32(kv_sm));
            for (int j = 0; j < nb && !*abort_p; ++j) {
                const int s = j % KV_STAGES, buf = j & 1;
                if (!mbar_wait(smem_u32(&bar_kv_full[s]), (j / KV_STAGES) & 1, abort_p)) break;
                if (j >= 2 && !mbar_wait(smem_u32(&bar_s_empty[buf]), ((j >> 1) & 1) ^ 1, abort_p)) break;
                tcgen05_fence_after();
                const uint64_t dk = dk0 + (uint64_t)(s * (kStageBytes >> 4));      // start addresses count 16 bytes
#pragma unroll
                for (int k = 0; k < D / 16; ++k)
                    umma_bf16(tmem_base + (uint32_t)(buf * TN), dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_s, k > 0 ? 1u : 0u);
                tcgen05_commit(smem_u32(&bar_s_full[buf]));
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------------------------------ issuer of O += P V
        if (lane == 0) {
            constexpr uint32_t idesc_o = instr_desc_mn(TM, D, true);
            const uint64_t dp0 = smem_desc_sw128(smem_u32(p_sm));
            const uint64_t dv0 = smem_desc_sw128_mn(smem_u32(kv_sm + 2 * kPageBytes));
            for (int j = 0; j < nb && !*abort_p; ++j) {
                const int s = j % KV_STAGES, buf = j & 1;
                if (!mbar_wait(smem_u32(&bar_kv_full[s]), (j / KV_STAGES) & 1, abort_p)) break;
                if (!mbar_wait(smem_u32(&bar_p_full[buf]), (j >> 1) & 1, abort_p)) break;
                tcgen05_fence_after();
                const uint64_t dp = dp0 + (uint64_t)(buf * (kPBytes >> 4));
                const uint64_t dv = dv0 + (uint64_t)(s * (kStageBytes >> 4));
#pragma unroll
                for (int k = 0; k < TN / 16; ++k) {
                    // P: K-major, 16 keys = 32 bytes along a row, the second 64 keys in the second half tile;
                    // V: MN-major, 16 keys = 16 rows of 128 bytes
                    umma_bf16(tmem_base + kColO + (uint32_t)(buf * D), dp + (uint64_t)((k >> 2) * ((TM * 128) >> 4) + (k & 3) * 2),
                              dv + (uint64_t)(k * ((16 * 128) >> 4)), idesc_o, (j >= 2 || k > 0) ? 1u : 0u);   // adds up over the group's blocks
                }
                tcgen05_commit(smem_u32(&bar_o_done[buf]));
                tcgen05_commit(smem_u32(&bar_kv_empty[s]));
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax, two threads a row
        // Warps 2-5 take the even blocks of keys, warps 6-9 the odd ones, for the same 128 rows (a warp reaches
        // the 32 lanes of tensor memory of its number modulo 4). Each group has its own S buffer, P buffer and
        // output accumulator in tensor memory and its own running maximum and sum, so the groups never wait for
        // each other: while one computes exponentials (16 a cycle an SM: the scarce unit) the other reads scores,
        // finds maxima or waits for its product. The two partial results of a row are merged once, at the end,
        // as key splits are merged in decoding.
        const int quarter = warp & 3, grp = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_col = (uint32_t)(grp * TN), o_col = kColO + (uint32_t)(grp * D);
        const int pos = r < rows_valid ? pos0 + r / G : -1;       // -1: the row sees nothing
        float m = -INFINITY, l = 0.0f;
        bool bad = false;                                         // a wait gave up: nothing more is waited for
        int done = 0;                                             // blocks this group has finished
        for (int j = grp; j < nb; j += 2, ++done) {
            if (!mbar_wait(smem_u32(&bar_s_full[grp]), done & 1, abort_p)) { bad = true; break; }
            tcgen05_fence_after();
            const int key0 = (b_lo + j) * TN;
            // a block that every row of the tile sees whole needs no test per key
            const bool plain = pos >= 0 && key0 + TN - 1 <= pos0 && (p.window == 0 || pos0 + nt - 1 - key0 < p.window);
            // this row's 128 scores of the block, read once and kept through both passes
            uint32_t raw[TN];
#pragma unroll
            for (int c = 0; c < TN; c += 32) tmem_ld32_nowait(lane_base + s_col + (uint32_t)c, raw + c);
            tmem_ld_wait();
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (plain) {
#pragma unroll
                for (int e = 0; e < TN; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(raw[e]));
            } else {
#pragma unroll
                for (int e = 0; e < TN; ++e) {
                    const int key = key0 + e;
                    const bool see = key <= pos && (p.window == 0 || pos - key < p.window);   // pos -1: nothing
                    if (!see) raw[e] = 0xff800000u;                // -inf: its weight will be exactly 0
                    mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(raw[e]));
                }
            }
            // the scale is positive: the largest scaled score is the scaled largest score
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            const float m_new = fmaxf(m, mx);
            const float mb = m_new == -INFINITY ? 0.0f : m_new;
            const float alpha = ex2(m - mb);                      // 0 while nothing was seen
            m = m_new;
            if (done >= 1 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                // The group's output so far lives in tensor memory, relative to the old maximum: rescale this row
                // before this block's P V adds to it. That product waits for this warp's arrival below, the one
                // before it is waited for here. The maximum of most later blocks does not move.
                if (!mbar_wait(smem_u32(&bar_o_done[grp]), (done - 1) & 1, abort_p)) { bad = true; break; }
                tcgen05_fence_after();
#pragma unroll 1
                for (int c = 0; c < D; c += 16) {                  // 16 columns at a time: the scores stay in registers
                    uint32_t acc[16];
                    tmem_ld16w(lane_base + o_col + (uint32_t)c, acc);
#pragma unroll
                    for (int e = 0; e < 16; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
                    tmem_st16w(lane_base + o_col + (uint32_t)c, acc);
                }
            }
            float add4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint8_t* p_row = p_sm + grp * kPBytes + r * 128;
#pragma unroll
            for (int i = 0; i < TN / 8; ++i) {                     // 8-key chunks; the second 64 keys in the second half tile
                float w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    w[e] = ex2(fmaf(__uint_as_float(raw[8 * i + e]), p.scale_log2, -mb));   // ex2(-inf) = 0
                    add4[e & 3] += w[e];
                }
                *reinterpret_cast<uint4*>(p_row + (i >> 3) * (TM * 128) + (((i & 7) ^ (r & 7)) << 4)) =
                    make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
            }
            l = l * alpha + ((add4[0] + add4[1]) + (add4[2] + add4[3]));
            fence_async_smem();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cta(smem_u32(&bar_p_full[grp]));
                mbar_arrive_cta(smem_u32(&bar_s_empty[grp]));
            }
        }
        // the group's output, once its last product is in
        float o[D];
#pragma unroll
        for (int d = 0; d < D; ++d) o[d] = 0.0f;
        if (!bad && done > 0) {
            if (mbar_wait(smem_u32(&bar_o_done[grp]), (done - 1) & 1, abort_p)) {
                tcgen05_fence_after();
                uint32_t acc[D];
                tmem_ld32_nowait(lane_base + o_col, acc);
                tmem_ld32_nowait(lane_base + o_col + 32, acc + 32);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < D; ++e) o[e] = __uint_as_float(acc[e]);
            } else {
                bad = true;
            }
        }
        // Every softmax thread comes here, whatever happened before, and learns whether anyone's wait gave up.
        // Past this barrier both groups' products are complete: P's memory is free for the merge.
        int any_bad;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "bar.red.or.pred p, 1, 256, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(any_bad) : "r"((int)bad) : "memory");
        float* merge = reinterpret_cast<float*>(p_sm);            // [D + 2][TM]: a thread's row is a column
        if (!any_bad && grp == 1) {
#pragma unroll
            for (int d = 0; d < D; ++d) merge[d * TM + r] = o[d];
            merge[D * TM + r] = m;                                // -inf and 0 when the group had no block
            merge[(D + 1) * TM + r] = l;
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (!any_bad && grp == 0 && r < rows_valid) {
            const float m1 = merge[D * TM + r], l1 = merge[(D + 1) * TM + r];
            const float mm = fmaxf(m, m1);
            const float mb = mm == -INFINITY ? 0.0f : mm;
            const float a0 = ex2(m - mb), a1 = ex2(m1 - mb);
            l = l * a0 + l1 * a1;
            const int t = tok_begin + t0 + r / G, h = kvh * G + r % G;
            float f = l > 0.0f ? 1.0f / l : 0.0f;
            if (p.gate != nullptr) f *= 1.0f / (1.0f + __expf(-__bfloat162float(p.gate[(int64_t)t * p.ld_gate + h])));
            const float f0 = a0 * f, f1 = a1 * f;
            uint4* dst = reinterpret_cast<uint4*>(p.out + ((int64_t)t * p.Hq + h) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = o[8 * c + e] * f0 + merge[(8 * c + e) * TM + r] * f1;
                dst[c] = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            }
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 1);
}

}  // namespace

// 1 when xs_attention_tc takes this problem: head size 64, pages of 64 keys, a group that divides 128.
XS_API int xs_attention_tc_supports(int D, int page_size, int G) {
    return D == 64 && page_size == PAGE && G >= 1 && G <= TM && TM % G == 0 && encode_fn() != nullptr;
}

// The same operation as xs_attention_mma with one key split, for prompts. pool: [pool_pages, 2, Hkv, 64, D].
// status: one device int that the kernel sets non-zero if a wait inside it gave up (the result is then invalid).
// max_kv_len: the longest sequence's keys, or 0 if the host does not know; it only picks the order in which CTAs start.
XS_API int xs_attention_tc(const void* q, const void* pool, int64_t pool_pages, const int32_t* page_table, int P,
                           const int32_t* cu_seqlens, const int32_t* kv_lens, const void* gate, int64_t ld_gate, void* out,
                           int T, int n_seqs, int max_q_len, int Hq, int Hkv, int D, int page_size, float scale, int window,
                           int max_kv_len, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: %d heads over %d kv heads", Hq, Hkv);
    const int G = Hq / Hkv;
    XS_REQUIRE(xs_attention_tc_supports(D, page_size, G),
               "attention (tcgen05): head size %d, page size %d, group %d is not supported", D, page_size, G);
    XS_REQUIRE(window >= 0 && max_q_len >= 1 && n_seqs >= 1 && P >= 1 && pool_pages >= 1 && status != nullptr,
               "attention (tcgen05): bad sizes");
    XS_REQUIRE(n_seqs <= 65535 && Hkv <= 65535, "attention (tcgen05): grid too large");
    XS_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)pool % 16 == 0 && (uintptr_t)out % 16 == 0,
               "attention (tcgen05): operands must be 16-byte aligned");
    alignas(64) CUtensorMap map;
    XS_REQUIRE(make_map(&map, pool, pool_pages * 2 * Hkv * PAGE, D, D, PAGE), "attention (tcgen05): the cache's tensor map could not be made");
    AttnTcParams p;
    p.q = (const __nv_bfloat16*)q;
    p.page_table = page_table;
    p.P = P;
    p.cu_seqlens = cu_seqlens;
    p.kv_lens = kv_lens;
    p.gate = (const __nv_bfloat16*)gate;
    p.ld_gate = ld_gate;
    p.out = (__nv_bfloat16*)out;
    p.status = status;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.G = G;
    p.tokens_per_tile = TM / G;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    // All kv heads of the latest tiles first (5 to 15 % faster up to 8,192 keys: the long tiles of every head start
    // before any short one) while the keys and values of all heads together stay well inside L2; one head after the
    // other beyond that (1.5 % faster at 32,000 keys).
    p.order = max_kv_len <= 0 || (int64_t)max_kv_len * Hkv * D * 4 <= (int64_t)32 << 20;
    const int max_tiles = ceil_div_i(max_q_len, p.tokens_per_tile);
    const size_t smem = (size_t)TM * D * 2 + (size_t)KV_STAGES * 4 * PAGE * D * 2 + 2 * (size_t)TM * TN * 2 + 1024;
    static bool opted = false;
    if (!opted) {
        cudaFuncSetAttribute(attention_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        opted = true;
    }
    const dim3 grid(max_tiles, n_seqs, Hkv);
    XS_REQUIRE(xs_launch(attention_tc_kernel<64>, grid, dim3(kAttnThreads), smem, stream, map, p) == cudaSuccess,
               "attention (tcgen05): launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}
