// out[M, N] = x[M, K] . w[N, K]^T for few rows (M <= 16): the decode-time matrix product.
//
// The weight is read exactly once, straight from HBM into registers (32-byte loads where nothing needs a predicate,
// 16-byte loads otherwise), and never staged: with M this small the product is bound by weight bandwidth. A CTA of 8 warps
// owns 16 weight rows and a slice of K; its warps take the slice's 32-wide k blocks in turn
// (warp w: blocks w, w+8, ...), four blocks' loads issued together. They multiply on tensor
// cores (mma.sync m16n8k16: weight rows on the M side, the batch on the N side) and add their
// partial sums in shared memory in warp order. A lane's 16 bytes are 8 consecutive k of one
// row; the same assignment of k to fragment slots is used for the weight and for x, which is
// all a contraction needs.
//
// What the activations cost (measured on B200, N 16384, K 2048, 8 rows, weights from memory, us): 14.3 with x read
// 16 bytes a lane; 12.0 with no x at all (the multiplies on zeros); 13.5 with 32 bytes a lane (a warp's load then
// covers whole lines of its 8 rows: half the trips through the load path, for x and for the weight); 12.9 with x asked
// for first thing after the wait and ahead of the next round's weights. Every CTA reads all of x for its 16 weight
// rows, 32 KB for 64 KB of weight; the multiplies themselves and the epilogue cost nothing measurable (mma.sync
// replaced by integer adds: the same time). A hint that asks a warp's later rounds of x into L1 right after the wait
// made the step slower (0.742 against 0.717 ms).
//
// Narrow outputs with a long K (the feed-forward's down projection) would leave most SMs
// idle, so K is cut into `ksplit` slices over blockIdx.y. Two to eight slices of a tile are the CTAs of one
// thread-block cluster: each puts its 16 x M sums into slice 0's shared memory, the cluster's barrier says that all
// have, and slice 0 adds them in slice order (no global memory, no counter; a slice more then costs 0.3 instead of
// 2.4 us). More slices than that: each slice's CTA writes its partial to scratch; the CTA that arrives last (a counter
// per row tile) adds the slices in slice order, so the sum does not depend on which CTA that was, and resets the counter.
//
// Epilogues: bias[N]; `residual` (float32 [M, N]) += result; or SwiGLU for a weight stacked in
// blocks of 8 gate rows and 8 up rows: out[M, N / 2] = silu(gate) * up.
//
// RMSNorm across the product (decode): a norm between two products is a kernel of its own only to wait in,
// so it is taken apart. The product that ends a branch adds its result to the float32 stream, and beside it
// leaves x~ = bfloat16(stream * next norm's weight) and, per row tile, the sum of squares of its 16 stream
// values per batch row (`next_*`, `out_ssq`). The product that follows reads x~, adds the tiles' sums in tile
// order and multiplies its result by 1 / sqrt(mean square + eps) per batch row (`in_ssq`): the scale is a
// factor per row of x, so it commutes with the contraction.
//
// The reference has the same split of work between its own kernel and a library: `gemv_t` up
// to 8 rows, oneMKL above (src/backend/sycl/sycl_kernels.cpp:630-714, sycl_kernels.h:280).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int ROWS = 16;      // weight rows per CTA
constexpr int UNROLL_DEFAULT = 4;     // k blocks whose loads a warp issues together
constexpr bool kBlocked = true;   // measured on B200: 3 % faster than interleaved on the wide shapes
constexpr int kSsqStaged = 128;  // producer tiles whose sums of squares are staged in shared memory
constexpr int K_PER_CTA = WARPS * UNROLL_DEFAULT * 32;   // a K slice this long is one round of loads per warp

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {   // weights are used once: do not keep them in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 32 bytes a lane: a warp's load covers whole 128-byte lines of 8 rows, half the trips through the load path of
// two 16-byte loads (sm_100 has 256-bit global loads).
__device__ __forceinline__ void ld_stream32(const void* p, uint4& lo, uint4& hi) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(p));
}
__device__ __forceinline__ void ld_act32(const void* p, uint4& lo, uint4& hi) {      // activations: kept in L1 for the SM's other CTAs
    asm volatile("ld.global.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(p));
}

struct SmallMParams {
    const __nv_bfloat16* x;
    const __nv_bfloat16* w;
    const float* bias;
    void* out;
    float* residual;
    float* partials;          // [tiles, ksplit, ROWS, 8 * NT] when ksplit > 1
    unsigned int* counters;   // [tiles], zero between calls
    int M, N, K, ksplit, swiglu, wave;
    int cluster;              // the K slices of a tile are the CTAs of one thread-block cluster: they meet in slice 0's shared memory
    int ragged;               // unpredicated instances: a K slice is a multiple of 64 but not of 1,024, so its last round is short
    int64_t ldx, ldw, ldo;
    // RMSNorm across the product (null / 0 when unused)
    const float* in_ssq;      // [in_tiles, 16]: sums of squares of x's stream rows, one row per producer tile
    int in_tiles, in_width;   // the stream's width (the mean's divisor)
    float in_eps;
    const float* next_w;      // [N]: the weight of the norm that reads the stream next
    __nv_bfloat16* next_x;    // [M, N]: bfloat16(stream * next_w)
    int64_t ld_next;
    float* out_ssq;           // [tiles, 16]
    // Gated short convolution behind the product (decode; null / 0 when unused): out is [M, 3 * conv_h] = [B | C | X]
    const float* conv_taps;   // [conv_k, conv_h]
    const float* conv_bias;   // [conv_h] or null
    __nv_bfloat16* conv_state;   // [slots, conv_k - 1, conv_h]
    const int32_t* conv_slots;   // [M]: batch row m's slot
    __nv_bfloat16* conv_out;     // [M, conv_h]
    unsigned int* conv_counters; // [conv_h / 16], zero between calls
    int conv_k, conv_h;
    // Per-head norm, rotation and cache write behind the product (an attention layer's q/k/v product in a decode step;
    // rope_q null when unused): out is [M, (Hq + 2 Hkv) D + ...] = [q heads | k heads | v heads | more]
    __nv_bfloat16* rope_q;          // [M, Hq, D]: normed, rotated queries
    __nv_bfloat16* rope_pool;       // [pages, 2, Hkv, page, D]: the cache; null: queries only (out is [q heads | more])
    const int32_t* rope_table;      // [n_seqs, rope_P] page numbers
    const int32_t* rope_seq;        // [M] sequence of a batch row
    const int32_t* rope_pos;        // [M] position of a batch row
    const float* rope_qw;           // [D] norm weights of q heads, or null: no norm
    const float* rope_kw;           // [D] of k heads
    const float2* rope_cs;          // [positions, D / 2] (cos, sin), or null: no rotation
    int rope_P, rope_hq, rope_hkv, rope_d, rope_page;
    float rope_eps;
    // Argmax of every batch row behind the product (the head; null when unused)
    unsigned long long* amax_keys;   // [16], zero between calls
    unsigned int* amax_counter;      // [1], zero between calls
    int32_t* amax_out;               // [M]
};

__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* p) {
    const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __bfloat162float(__ushort_as_bfloat16(raw));
}

// The convolution that follows in_proj, inside the product's kernel. The three CTAs that own a group of 16 channels
// (its B, its C and its X rows: tiles g, g + H / 16, g + 2 H / 16) are one thread-block cluster (the kernel maps
// blockIdx.x to tiles that way); the C and the X CTA put their values into the B CTA's shared memory, the cluster's
// barrier says that they have, and the B CTA finishes: every sequence brings one token (batch row m is sequence m),
// g = bfloat16(B * X); out = C * (bias + sum_j tap_j * state_j + tap_last * g); the state moves up by one row and takes
// g. The same arithmetic on the same rounded values, in the same order, as the kernel of its own (short_conv.cu), so a
// sequence's values do not depend on which of them ran. (Every CTA said at its start that it runs: the first cluster
// barrier's arrival; nobody writes into another's shared memory before it has seen that.)
template <int NT>
__device__ __forceinline__ void conv_tail(const SmallMParams& p, const float (*sum)[8 * NT + 1], const float* inv, int n0) {
    __shared__ float cx[2][ROWS][8 * NT + 1];
    const int rank = (int)(blockIdx.x % 3u), group = (int)(blockIdx.x / 3u);
    const int H = p.conv_h, K = p.conv_k;
    const int i = threadIdx.x;
    const int r = i % ROWS, m = i / ROWS;
    const bool mine = i < ROWS * 8 * NT && m < p.M;
    float v = 0.0f;
    if (mine) {
        v = sum[r][m] * inv[m];
        if (p.bias != nullptr) v += p.bias[n0 + r];
        v = __bfloat162float(__float2bfloat16_rn(v));          // as the stored [B | C | X] holds it
    }
    // the leader's own loads do not wait for the others
    const int c = group * ROWS + r;
    __nv_bfloat16* st = nullptr;
    float acc = 0.0f;
    __nv_bfloat16 old[7];
    if (rank == 0 && mine) {
        st = p.conv_state + (int64_t)p.conv_slots[m] * (K - 1) * H + c;
        acc = p.conv_bias != nullptr ? p.conv_bias[c] : 0.0f;
#pragma unroll
        for (int j = 0; j < 7; ++j)
            if (j < K - 1) old[j] = st[(int64_t)j * H];
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");              // all three have started
    if (rank != 0 && mine) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(&cx[rank - 1][r][m])));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank != 0 || !mine) return;
    const float gate = cx[0][r][m], x = cx[1][r][m];
    const __nv_bfloat16 g16 = __float2bfloat16_rn(v * x);
    const float g = __bfloat162float(g16);
#pragma unroll
    for (int j = 0; j < 7; ++j) {
        if (j < K - 1) {
            acc = fmaf(p.conv_taps[(int64_t)j * H + c], __bfloat162float(old[j]), acc);
            if (j > 0) st[(int64_t)(j - 1) * H] = old[j];        // row j moves to j - 1
        }
    }
    acc = fmaf(p.conv_taps[(int64_t)(K - 1) * H + c], g, acc);
    st[(int64_t)(K - 2) * H] = g16;
    p.conv_out[(int64_t)m * H + c] = __float2bfloat16_rn(acc * gate);
}

// An attention layer's q/k/v product in a decode step, finished inside the product's kernel: the D / 16 CTAs that own
// a head's rows are one thread-block cluster (heads lie one after another in the output, so they are neighbours). Every
// CTA rounds its 16 x M values as the stored output holds them, sends its sums of squares to all CTAs of the head and
// its values to the CTA that owns the other half of its rotation pairs (i and i + D / 2), and after the cluster's
// barrier finishes its own 16 channels: RMSNorm over the head (q and k heads), rotation by the position's (cos, sin),
// then the queries go to rope_q and keys and raw values into the cache's page, as qk_norm_rope_store (the kernel of
// its own, attention_generic.cu) does. Tiles behind the heads (the head gate's rows) take no part.
template <int NT>
__device__ __forceinline__ void rope_tail(const SmallMParams& p, const float (*sum)[8 * NT + 1], const float* inv, int n0) {
    __shared__ float part_ss[8][8 * NT];                  // [quarter of the head][batch row]
    __shared__ float partner[ROWS][8 * NT + 1];
    const int D = p.rope_d, per_head = D / ROWS;
    const int heads = p.rope_hq + (p.rope_pool != nullptr ? 2 * p.rope_hkv : 0);
    const int tile = n0 / ROWS;
    if (tile >= heads * per_head) return;                 // (whole clusters: heads * per_head is a multiple of per_head)
    const int hh = tile / per_head, qd = tile % per_head, half_q = per_head / 2;
    const int which = hh < p.rope_hq ? -1 : (hh - p.rope_hq) / p.rope_hkv;      // -1 q, 0 k, 1 v
    const float* w = which < 0 ? p.rope_qw : which == 0 ? p.rope_kw : nullptr;
    const bool rotate = which <= 0 && p.rope_cs != nullptr;
    const int i = threadIdx.x, r = i % ROWS, m = i / ROWS;
    const bool mine = i < ROWS * 8 * NT && m < p.M;
    float v = 0.0f;
    if (mine) {
        v = sum[r][m] * inv[m];
        if (p.bias != nullptr) v += p.bias[n0 + r];
        v = __bfloat162float(__float2bfloat16_rn(v));
    }
    // what does not wait for the others: the position's (cos, sin), the norm weights, where the result goes
    const int dim = qd * ROWS + r, pair = dim % (D / 2);
    float2 cs = make_float2(1.0f, 0.0f);
    float w_own = 1.0f, w_other = 1.0f;
    __nv_bfloat16* dst = nullptr;
    if (mine) {
        const int pos = p.rope_pos[m];
        if (rotate) cs = p.rope_cs[(int64_t)pos * (D / 2) + pair];
        if (w != nullptr) {
            w_own = w[dim];
            w_other = w[dim < D / 2 ? dim + D / 2 : dim - D / 2];
        }
        if (which < 0) {
            dst = p.rope_q + ((int64_t)m * p.rope_hq + hh) * D + dim;
        } else {
            const int kvh = (hh - p.rope_hq) % p.rope_hkv;
            const int page = p.rope_table[(int64_t)p.rope_seq[m] * p.rope_P + pos / p.rope_page];
            dst = p.rope_pool + ((((int64_t)page * 2 + which) * p.rope_hkv + kvh) * p.rope_page + pos % p.rope_page) * D + dim;
        }
    }
    // sums of squares of this CTA's 16 channels per batch row: the 16 lanes of a row's channels sit side by side
    float sq = v * v;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");              // every CTA of the head has started
    if (mine) {
        if (r == 0) {
            for (int c = 0; c < per_head; ++c) {
                uint32_t at;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(at) : "r"((uint32_t)__cvta_generic_to_shared(&part_ss[qd][m])), "r"(c));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(at), "f"(sq) : "memory");
            }
        }
        if (rotate) {
            uint32_t at;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(at) : "r"((uint32_t)__cvta_generic_to_shared(&partner[r][m])),
                         "r"(qd < half_q ? qd + half_q : qd - half_q));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(at), "f"(v) : "memory");
        }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (!mine) return;
    float x = v, y = rotate ? partner[r][m] : 0.0f;
    if (w != nullptr) {
        float ss = 0.0f;
        for (int c = 0; c < per_head; ++c) ss += part_ss[c][m];
        const float scale = 1.0f / sqrtf(ss / (float)D + p.rope_eps);
        x = x * scale * w_own;
        y = y * scale * w_other;
    }
    if (rotate) x = dim < D / 2 ? x * cs.x - y * cs.y : x * cs.x + y * cs.y;
    *dst = __float2bfloat16_rn(x);
}

// Each batch row's largest output and its column, the lowest column among equals: every CTA folds its 16 columns into one
// 64-bit key per batch row (the value's bits made monotone, then the column counted down), the keys meet by atomicMax,
// and the CTA that stores last unpacks them and clears them for the next call.
template <int NT>
__device__ __forceinline__ void argmax_tail(const SmallMParams& p, const float (*sum)[8 * NT + 1], const float* inv, int n0) {
    __shared__ bool is_last;
    if (threadIdx.x < 8 * NT && (int)threadIdx.x < p.M) {
        const int m = threadIdx.x;
        float best = -INFINITY;
        int at = -1;
        for (int r = 0; r < ROWS; ++r) {
            const int n = n0 + r;
            if (n >= p.N) break;
            float v = sum[r][m] * inv[m];               // the value as it was stored
            if (p.bias != nullptr) v += p.bias[n];
            if (v > best || at < 0) {
                best = v;
                at = n;
            }
        }
        if (at >= 0) {
            unsigned int u = __float_as_uint(best);
            u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            atomicMax(&p.amax_keys[m], ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)at));
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(p.amax_counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if ((int)threadIdx.x < p.M) {
        const unsigned long long key = atomicExch(&p.amax_keys[threadIdx.x], 0ull);
        p.amax_out[threadIdx.x] = (int32_t)(0xFFFFFFFFu - (unsigned int)(key & 0xFFFFFFFFull));
    }
    if (threadIdx.x == 0) *p.amax_counter = 0;
}

// `staged` (8 batch rows only): this tile's old stream values [m][16] and the next norm's weights [16], fetched into
// shared memory while the weights streamed, so that the CTA's tail does not begin with a trip to L2.
// TAIL: what runs behind the product in its kernel (0 nothing, 1 the short convolution, 2 the heads' norm, rotation and
// cache write, 3 the argmax): instances of their own, so that the products without a tail do not carry its registers.
template <int NT, typename TO, int TAIL>
__device__ __forceinline__ void epilogue(const SmallMParams& p, const float (*sum)[8 * NT + 1], const float* inv, int n0,
                                         const float* staged = nullptr) {
    TO* out = reinterpret_cast<TO*>(p.out);
    if (p.swiglu) {
        // rows 0..7 of the tile are gate rows, rows 8..15 the up rows of the same outputs
        for (int i = threadIdx.x; i < 8 * 8 * NT; i += WARPS * 32) {
            const int r = i % 8, m = i / 8;
            if (m >= p.M || n0 + 8 + r >= p.N) continue;
            float gate = sum[r][m] * inv[m], up = sum[r + 8][m] * inv[m];
            if (p.bias != nullptr) {
                gate += p.bias[n0 + r];
                up += p.bias[n0 + 8 + r];
            }
            out[(int64_t)m * p.ldo + (n0 >> 1) + r] = from_f32<TO>(gate / (1.0f + expf(-gate)) * up);
        }
        return;
    }
    // ROWS * 8 * NT is 128 or 256: whole warps enter, once
    for (int i = threadIdx.x; i < ROWS * 8 * NT; i += WARPS * 32) {
        const int r = i % ROWS, m = i / ROWS;       // neighbouring threads write neighbouring columns of out
        const int n = n0 + r;
        const bool live = m < p.M && n < p.N;
        float v = sum[r][m] * inv[m];
        if (live && p.bias != nullptr) v += p.bias[n];
        float sq = 0.0f;
        if (live) {
            if (p.residual != nullptr) {
                const float old = staged != nullptr ? staged[m * ROWS + r] : p.residual[(int64_t)m * p.ldo + n];
                const float h = old + v;
                p.residual[(int64_t)m * p.ldo + n] = h;
                if (p.next_x != nullptr) {
                    const float nw = staged != nullptr ? staged[8 * ROWS + r] : p.next_w[n];
                    p.next_x[(int64_t)m * p.ld_next + n] = __float2bfloat16_rn(h * nw);
                }
                sq = h * h;
            } else {
                out[(int64_t)m * p.ldo + n] = from_f32<TO>(v);
            }
        }
        if (p.out_ssq != nullptr) {     // the tile's 16 columns of batch row m sit in 16 neighbouring lanes
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (r == 0) p.out_ssq[(int64_t)blockIdx.x * 16 + m] = sq;
        }
    }
    if (TAIL == 1) conv_tail<NT>(p, sum, inv, n0);
    if (TAIL == 2) rope_tail<NT>(p, sum, inv, n0);
    if (TAIL == 3) argmax_tail<NT>(p, sum, inv, n0);
}

// EXACT: N is a multiple of 16 and every K slice a multiple of 64 (of 1,024 = 8 warps x 4 blocks x 32 unless `ragged`), so no row is
// clamped and no load is predicated: a third fewer instructions in the loop that feeds the memory system.
// UNROLL 8 (EXACT only, K slices that are multiples of 2,048): sixteen loads a lane in flight instead of eight, so a
// slice of 2,048 is one round, all of it requested before the wait for the previous kernel; twice the registers
// for weights, two CTAs an SM instead of four. For grids of at most one such wave (the narrow outputs, which are
// bound by latency, not bandwidth): measured on the whole decode step, 1.2B shape, batch 8: 0.811 -> 0.773 ms with
// it on the attention and convolution output projections and the q/k/v product; on grids of more CTAs it loses.
template <int NT, typename TO, bool EXACT, int UNROLL = UNROLL_DEFAULT, int TAIL = 0>
__global__ void __launch_bounds__(WARPS * 32, UNROLL == 4 ? ((NT == 2 && EXACT) ? 3 : 4) : 2) gemm_small_m_kernel(const SmallMParams p) {
    __shared__ float red[WARPS][ROWS][8 * NT + 1];
    __shared__ float sum[ROWS][8 * NT + 1];
    __shared__ __align__(16) float ssq_in[kSsqStaged][16];
    __shared__ float ssq_red[WARPS][17];
    __shared__ float inv[16];
    __shared__ __align__(16) float staged[9 * ROWS];      // old stream values [8][16], then the next norm's weights [16]
    __shared__ bool last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    // (with the convolution behind the product, three neighbouring CTAs are the B, C and X tiles of one group of channels)
    const int tile = TAIL == 1 ? (int)(blockIdx.x % 3u) * (p.conv_h / ROWS) + (int)(blockIdx.x / 3u) : (int)blockIdx.x;
    const int slice = blockIdx.y;
    // K slices as one cluster (see the reduction below): a CTA may write to another's shared memory only when that one
    // has started; every CTA says so here, first thing, and looks for the others' word just before it writes
    const bool clustered = p.ksplit > 1 && p.cluster;
    // (with the rotation behind the product the grid is rounded up to whole clusters: CTAs past the last tile leave; the
    // tiles of a head are a cluster that meets, those behind the heads do not)
    if (TAIL == 2 && tile * ROWS >= p.N) return;
    const bool rope_head = TAIL == 2 && tile < (p.rope_hq + (p.rope_pool != nullptr ? 2 * p.rope_hkv : 0)) * (p.rope_d / ROWS);
    if (clustered || TAIL == 1 || rope_head) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const int n0 = tile * ROWS;
    // clamped: out-of-range rows are not stored
    const int ra = EXACT ? n0 + g : min(n0 + g, p.N - 1), rb = EXACT ? n0 + g + 8 : min(n0 + g + 8, p.N - 1);
    // EXACT: a lane takes 16 consecutive k (32 bytes) of a row at a time, which fill the fragment slots of two
    // neighbouring 32-wide k blocks; otherwise 8 (16 bytes) of one block. Weights and x use the same assignment.
    static_assert(kBlocked, "pairs of neighbouring k blocks");
    constexpr int kLane = EXACT ? 16 : 8;
    const __nv_bfloat16* wa_p = p.w + (int64_t)ra * p.ldw + q * kLane;
    const __nv_bfloat16* wb_p = p.w + (int64_t)rb * p.ldw + q * kLane;
    const __nv_bfloat16* x_p[NT];
    bool x_ok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        x_ok[t] = t * 8 + g < p.M;
        x_p[t] = p.x + (int64_t)(x_ok[t] ? t * 8 + g : 0) * p.ldx + q * kLane;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;

    // this CTA's k blocks: [kb_begin, kb_end); this warp takes every WARPS-th of them
    const int k_blocks = (p.K + 31) / 32;
    const int per_slice = (k_blocks + p.ksplit - 1) / p.ksplit;
    const int kb_begin = slice * per_slice, kb_end = min(k_blocks, kb_begin + per_slice);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // The first round of weight loads depends on no other kernel: it is issued before pdl_wait(), so
    // that the weights are already on their way while the previous kernel of the step finishes.
    pdl_launch_dependents();
    uint4 wa[UNROLL], wb[UNROLL];
    // k blocks of a round: warp w takes blocks w*ws + u*us. blocked (ws = 4, us = 1): a warp's four loads
    // cover 256 consecutive bytes of a row; interleaved (ws = 1, us = WARPS): the CTA's warps cover them together.
    // Sixteen loads a round are two rounds of eight in one (slots 4..7 are the warp's blocks of the next 32 of the
    // CTA), so that a warp adds up the same blocks in the same order in both variants: a row's bits do not depend on
    // which variant its batch or its shape chose.
    constexpr int ws = kBlocked ? UNROLL_DEFAULT : 1, us = kBlocked ? 1 : WARPS;
    auto slot = [](int u) { return (u / UNROLL_DEFAULT) * (WARPS * UNROLL_DEFAULT) + (u % UNROLL_DEFAULT) * us; };
    int kb = kb_begin + warp * ws;
    // (unpredicated instances: a pair of k blocks is all inside the slice or all outside, the same for every lane of
    // the warp, and only a slice whose length is no multiple of 1,024 has pairs outside, in its last round)
    auto load_w32 = [&](int at) {
#pragma unroll
        for (int u = 0; u < UNROLL; u += 2) {
            if (!p.ragged || at + slot(u) < kb_end) {
                ld_stream32(wa_p + (at + slot(u)) * 32, wa[u], wa[u + 1]);
                ld_stream32(wb_p + (at + slot(u)) * 32, wb[u], wb[u + 1]);
            } else {
                wa[u] = wa[u + 1] = wb[u] = wb[u + 1] = zero;
            }
        }
    };
    if (EXACT) {
        load_w32(kb);
    } else {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k0 = (kb + slot(u)) * 32;
            // K is a multiple of 8: a lane's 8 elements are all inside or all outside
            const bool in = kb + slot(u) < kb_end && k0 + q * 8 < p.K;
            wa[u] = in ? ld_stream(wa_p + k0) : zero;
            wb[u] = in ? ld_stream(wb_p + k0) : zero;
        }
    }
    if (kBlocked) {
        // The rounds after the first are asked into L2 now (a hint, no registers held): when their loads are
        // issued after the first round's multiplies they find the lines on the chip. A warp's round is 256
        // consecutive bytes (sixteen loads: two such pieces) of each of its 16 rows: lane -> (row, which 128-byte line).
        const int prow = min(n0 + (lane & 15), p.N - 1);
        const __nv_bfloat16* pbase = p.w + (int64_t)prow * p.ldw + (lane >> 4) * 64;
#pragma unroll 1
        for (int r = 1; r <= 3; ++r) {
            const int pkb = kb + r * WARPS * UNROLL;
#pragma unroll
            for (int h = 0; h < UNROLL / UNROLL_DEFAULT; ++h) {
                const int hkb = pkb + h * WARPS * UNROLL_DEFAULT;
                if (hkb < kb_end && hkb * 32 + (lane >> 4) * 64 < p.K)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(pbase + (int64_t)hkb * 32));
            }
        }
        // More row tiles than CTAs that fit on the chip at once: also ask for the first round of the tile
        // that will take this CTA's place (CTAs start in index order, `wave` of them at a time).
        const int later = tile + p.wave;
        if (p.wave > 0 && later < (int)gridDim.x) {
            const int lrow = min(later * ROWS + (lane & 15), p.N - 1);
            if (kb < kb_end && kb * 32 + (lane >> 4) * 64 < p.K)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w + (int64_t)lrow * p.ldw + (lane >> 4) * 64 + (int64_t)kb * 32));
        }
    }
    pdl_wait();
    uint4 xv[UNROLL][NT];
    auto load_x32 = [&](int at) {
#pragma unroll
        for (int u = 0; u < UNROLL; u += 2) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (x_ok[t] && (!p.ragged || at + slot(u) < kb_end)) ld_act32(x_p[t] + (at + slot(u)) * 32, xv[u][t], xv[u + 1][t]);
                else xv[u][t] = xv[u + 1][t] = zero;
            }
        }
    };
    // Up to 8 batch rows, the first round's x is asked for first thing after the wait, and the next round's right after
    // this round's multiplies, ahead of the next round's weights: it comes from L1 or L2 and should not queue behind
    // loads from memory (measured on B200, whole decode step, 1.2B shape, batch 8: 0.709 -> 0.687 ms; batch 1: 0.649 ->
    // 0.635). With 16 rows the registers do not allow it.
    constexpr bool kXAhead = EXACT && NT == 1;
    if (kXAhead) load_x32(kb);
    // the stream values this tile will be added to, and the next norm's weights, travel to shared memory beside the
    // main loop too (whole tiles of up to 8 batch rows only)
    const bool stage_tail = NT == 1 && EXACT && p.residual != nullptr && !p.swiglu;
    if (stage_tail) {
        const int i = threadIdx.x;
        if (i < 8 * ROWS) {
            const int m = i / ROWS, r = i % ROWS;
            if (m < p.M)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(&staged[i])),
                             "l"(p.residual + (int64_t)m * p.ldo + n0 + r) : "memory");
        } else if (i < 9 * ROWS && p.next_w != nullptr) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(&staged[i])),
                         "l"(p.next_w + n0 + (i - 8 * ROWS)) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // the producer's per-tile sums of squares travel to shared memory beside the main loop (no registers held,
    // nothing waits for them until the first round's multiplies are done): a thread asks for the 16-byte chunks
    // (a tile's sums of 4 batch rows) that it will add up itself, and only those of rows the batch has
    const int ssq_rows = (threadIdx.x & 3) * 4;          // this thread's batch rows: ssq_rows .. ssq_rows + 3
    const bool ssq_mine = p.in_ssq != nullptr && ssq_rows < p.M;
    if (ssq_mine) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = threadIdx.x + WARPS * 32 * u;          // 16-byte chunk: tile c / 4, batch rows (c % 4) * 4 ...
            if ((c >> 2) < p.in_tiles)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&ssq_in[c >> 2][(c & 3) * 4])),
                             "l"(p.in_ssq + (int64_t)c * 4) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // The sums of squares are added up behind the main loop without a barrier of their own: a thread adds the chunks
    // it asked for itself (tiles t and t + 64, then every 64th beyond the staged ones), the lanes of a warp that hold
    // the same batch rows meet by shuffles, and the warps' sums wait in shared memory for the barrier that the
    // reduction of the products needs anyway. Fixed order: no sum depends on timing. (Measured on B200, N 16384,
    // K 2048, 8 rows: the carried norm costs its consumer 1.0 of 14.6 us: 0.5 the loads, 0.7 these sums, 0.4 the
    // rows' 1 / rms, not additive; done after the first round's multiplies instead: the same or slightly slower.)
    auto ssq_first_level = [&]() {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (ssq_mine) {
            asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = threadIdx.x + WARPS * 32 * u;
                if ((c >> 2) < p.in_tiles) {
                    const float4 a = *reinterpret_cast<const float4*>(&ssq_in[c >> 2][ssq_rows]);
                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                }
            }
            for (int t = kSsqStaged + (threadIdx.x >> 2); t < p.in_tiles; t += WARPS * 8) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(p.in_ssq + (int64_t)t * 16 + ssq_rows));
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
            v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
            v.z += __shfl_xor_sync(0xffffffffu, v.z, o);
            v.w += __shfl_xor_sync(0xffffffffu, v.w, o);
        }
        if (lane < 4) {
            ssq_red[warp][lane * 4 + 0] = v.x;
            ssq_red[warp][lane * 4 + 1] = v.y;
            ssq_red[warp][lane * 4 + 2] = v.z;
            ssq_red[warp][lane * 4 + 3] = v.w;
        }
    };
    for (; kb - warp * ws < kb_end; kb += WARPS * UNROLL) {
        if (EXACT && !kXAhead) load_x32(kb);
        if (!EXACT) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int k0 = (kb + slot(u)) * 32;
                const bool in = kb + slot(u) < kb_end && k0 + q * 8 < p.K;
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    xv[u][t] = (in && x_ok[t]) ? *reinterpret_cast<const uint4*>(x_p[t] + k0) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                mma_bf16_16816(acc[t], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv[u][t].x, xv[u][t].y);
                mma_bf16_16816(acc[t], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv[u][t].z, xv[u][t].w);
            }
        }
        const int nkb = kb + WARPS * UNROLL;      // the next round's weights
        if (EXACT) {
            if (nkb - warp * ws < kb_end) {       // the same for the whole CTA
                if (kXAhead) load_x32(nkb);
                load_w32(nkb);
            }
        } else {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int k0 = (nkb + slot(u)) * 32;
                const bool in = nkb + slot(u) < kb_end && k0 + q * 8 < p.K;
                wa[u] = in ? ld_stream(wa_p + k0) : zero;
                wb[u] = in ? ld_stream(wb_p + k0) : zero;
            }
        }
    }
    if (p.in_ssq != nullptr) ssq_first_level();
    // c0, c1: (weight row g, batch q * 2 + {0, 1}); c2, c3: weight row g + 8
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        red[warp][g][t * 8 + q * 2] = acc[t][0];
        red[warp][g][t * 8 + q * 2 + 1] = acc[t][1];
        red[warp][g + 8][t * 8 + q * 2] = acc[t][2];
        red[warp][g + 8][t * 8 + q * 2 + 1] = acc[t][3];
    }
    // Several K slices as one cluster (2 to 8 of them): every slice puts its sums straight into slice 0's shared memory
    // (its own place there), the cluster's barrier says that all have, and slice 0 adds them in slice order. No global
    // memory, no fence, no counter; nobody polls.
    __shared__ float parts[8][ROWS][8 * NT + 1];
    uint32_t remote = 0;
    if (clustered) {
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");          // (all have started: long true)
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(&parts[slice][0][0])));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ROWS * 8 * NT; i += WARPS * 32) {
        const int r = i / (8 * NT), m = i % (8 * NT);
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) v += red[wv][r][m];
        if (clustered) asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((r * (8 * NT + 1) + m) * 4)), "f"(v) : "memory");
        else sum[r][m] = v;
    }
    if (threadIdx.x >= WARPS * 32 - 16) {      // the last 16 threads (idle above for up to 8 rows): each batch row's 1 / rms
        const int m = threadIdx.x - (WARPS * 32 - 16);
        float v = 1.0f;
        if (p.in_ssq != nullptr) {
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < WARPS; ++j) ss += ssq_red[j][m];
            v = 1.0f / sqrtf(ss / (float)p.in_width + p.in_eps);
        }
        inv[m] = v;
    }
    if (stage_tail) asm volatile("cp.async.wait_all;" ::: "memory");      // (this thread's; the barrier below shows them to all)
    if (clustered) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (slice != 0) return;
        for (int i = threadIdx.x; i < ROWS * 8 * NT; i += WARPS * 32) {
            float v = 0.0f;
            for (int s = 0; s < p.ksplit; ++s) v += parts[s][i / (8 * NT)][i % (8 * NT)];     // slice order
            sum[i / (8 * NT)][i % (8 * NT)] = v;
        }
        __syncthreads();
        epilogue<NT, TO, TAIL>(p, sum, inv, n0, stage_tail ? staged : nullptr);
        return;
    }
    __syncthreads();
    if (p.ksplit == 1) {
        epilogue<NT, TO, TAIL>(p, sum, inv, n0, stage_tail ? staged : nullptr);
        return;
    }
    // ---- more slices than a cluster holds: leave this slice's partial, and let the last CTA to arrive add them all
    float* mine = p.partials + ((int64_t)tile * p.ksplit + slice) * (ROWS * 8 * NT);
    for (int i = threadIdx.x; i < ROWS * 8 * NT; i += WARPS * 32) mine[i] = sum[i / (8 * NT)][i % (8 * NT)];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&p.counters[tile], 1u) == (unsigned)p.ksplit - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    const float* all = p.partials + (int64_t)tile * p.ksplit * (ROWS * 8 * NT);
    for (int i = threadIdx.x; i < ROWS * 8 * NT; i += WARPS * 32) {
        float v = 0.0f;
        for (int s = 0; s < p.ksplit; ++s) v += __ldcg(all + (int64_t)s * (ROWS * 8 * NT) + i);   // slice order
        sum[i / (8 * NT)][i % (8 * NT)] = v;
    }
    if (threadIdx.x == 0) p.counters[tile] = 0;    // ready for the next call
    __syncthreads();
    epilogue<NT, TO, TAIL>(p, sum, inv, n0, stage_tail ? staged : nullptr);
}

}  // namespace

// CTAs of this kernel that are resident on the device at once (4 an SM); 0 until the first launch asks the device.
int g_small_m_wave = 0;

XS_API int xs_gemm_small_m_supports(int M, int K, int64_t ldx, int64_t ldw) {
    return M >= 1 && M <= 16 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

int g_small_m_ksplit_max = 4;
XS_API void xs_gemm_small_m_set_ksplit_max(int n) { g_small_m_ksplit_max = n; }
int g_small_m_cluster = 1;        // K slices (2 to 8) of a tile as one thread-block cluster
XS_API void xs_gemm_small_m_set_cluster(int on) { g_small_m_cluster = on; }
int g_small_m_one_round = 1;      // 0: off; 1: on, for grids of at most two CTAs an SM; n > 1: for grids of at most n CTAs
XS_API void xs_gemm_small_m_set_one_round(int on) { g_small_m_one_round = on; }

// How many K slices the kernel would like for this shape on a device with `sms` SMs, and the
// scratch (bytes) that needs: partial sums, then one counter per row tile. 0 bytes when 1 slice.
XS_API int xs_gemm_small_m_ksplit(int M, int N, int K, int sms) {
    // Measured on B200 inside a CUDA graph (M 8, us). With the slices of a tile as one cluster that meets in shared
    // memory: N 2048, K 8192: 9.2 in one slice, 7.7 in two, 7.3 in four, 9.5 in eight; N 2048, K 2048: 2.5, 3.4, 3.5;
    // N 3072, K 2048: 3.0, 3.8; N 6144, K 2048: 5.1, 7.9; N 2048, K 10752: 14.6, 12.4, 10.5 (three), 9.8 (four), 11.5
    // (six). (With scratch memory and a counter instead, a slice more cost 2.4 us: 8.6, 8.6, 9.1 for the first shape,
    // 2.5 against 4.9 for the second.) So: one slice for K up to 2,048 and for outputs wide enough to fill the device
    // twice; otherwise about 2,048 of K a slice, at most `ksplit_max` slices and at most four CTAs an SM, and slices
    // that the unpredicated instances take (whole pairs of k blocks) where there are such.
    const int tiles = ceil_div_i(N, ROWS);
    if (tiles >= 2 * sms) return 1;
    int ks = K / 2048;                // at least 2048 of K a slice
    if (ks > g_small_m_ksplit_max) ks = g_small_m_ksplit_max;
    while (ks > 1 && (int64_t)tiles * ks > 4 * (int64_t)sms) --ks;
    if (ks < 1) ks = 1;
    if (N % ROWS == 0)
        for (int k2 = ks; k2 > 1; --k2)
            if (K % k2 == 0 && (K / k2) % 64 == 0) return k2;
    return ks;
}

// Scratch layout: partial sums from the front; the last kCounterBytes hold one counter per row tile.
constexpr int64_t kCounterBytes = 65536;

XS_API int64_t xs_gemm_small_m_scratch_bytes(int M, int N, int ksplit) {
    if (ksplit <= 1) return 0;
    const int64_t tiles = ceil_div_i(N, ROWS);
    const int nt = M <= 8 ? 1 : 2;
    return tiles * ksplit * ROWS * 8 * nt * (int64_t)sizeof(float) + kCounterBytes;
}

// x, w bfloat16; out bfloat16 or float32 (out_dtype), or residual += when `residual` is given (float32, stride ldo).
// swiglu != 0: w holds blocks of 8 gate rows and 8 up rows; out is [M, N / 2] = silu(gate) * up.
// ksplit > 1 needs `scratch` of at least xs_gemm_small_m_scratch_bytes. Its last 64 KiB are the counters: zero
// before the first call, and zero again whenever the kernel has run; a caller that keeps one buffer for all
// shapes passes the whole buffer every time, so that the counters stay in the same place.
//
// RMSNorm across the product (see the top of this file), all optional:
//   in_ssq [in_tiles, 16], in_width, in_eps: x is x~ of a stream whose rows' sums of squares a producer left per
//     tile; the result is scaled by 1 / sqrt(sum / in_width + in_eps) per batch row (before the bias).
//   next_w [N], next_x [M, N] bfloat16 (stride ld_next), out_ssq [ceil(N / 16), 16]: with `residual`, also leave
//     bfloat16(stream * next_w) and this product's per-tile sums of squares of the new stream values.
//
// Work that follows the product in the same kernel, by the CTA that finishes last (nobody waits), all optional:
//   conv_*: the product is a short-convolution layer's in_proj for one token a sequence (out bfloat16 [M, 3 H] = [B | C | X],
//     one K slice, H a multiple of 16): the gated convolution over each sequence's state (conv_state [slots, taps - 1, H],
//     conv_slots [M]) goes to conv_out [M, H] and the state moves on. conv_counters: H / 16 zeroed words, left zeroed.
//   amax_*: amax_out [M] takes each batch row's column of the largest output (the lowest among equals); amax_keys:
//     16 zeroed 64-bit words and amax_counter one zeroed word, left zeroed.
//   rope (xs_gemm_small_m_rope): the product is an attention layer's q/k/v product for one token a sequence (out bfloat16
//     [M, (Hq + 2 Hkv) D + more], or [M, Hq D + more] without a cache to write; D 32, 64 or 128; one K slice): per-head
//     RMSNorm (q_w, k_w: [D] or null), rotation (cs: [positions, D / 2, 2] or null), queries to q_out [M, Hq, D], keys
//     and raw values into the cache's pages, as xs_qk_norm_rope_store does.
struct XsRopeTail {
    void* q_out;
    void* pool;
    const int32_t* page_table;
    const int32_t* seq_of_token;
    const int32_t* positions;
    const float* q_w;
    const float* k_w;
    const float* cs;
    int P, Hq, Hkv, D, page_size;
    float eps;
};

static int small_m_launch(const void* x, const void* w, const float* bias, void* out, float* residual,
                          int out_dtype, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int swiglu,
                          int ksplit, void* scratch, int64_t scratch_bytes, const float* in_ssq, int in_tiles,
                          int in_width, float in_eps, const float* next_w, void* next_x, int64_t ld_next,
                          float* out_ssq, const float* conv_taps, const float* conv_bias, void* conv_state,
                          const int32_t* conv_slots, void* conv_out, void* conv_counters, int conv_k, int conv_h,
                          void* amax_keys, void* amax_counter, int32_t* amax_out, const XsRopeTail* rope,
                          cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    XS_REQUIRE(rope == nullptr ||
                   (rope->q_out != nullptr && rope->positions != nullptr && rope->seq_of_token != nullptr &&
                    (rope->D == 32 || rope->D == 64 || rope->D == 128) && rope->Hq > 0 && rope->Hkv > 0 &&
                    (rope->pool == nullptr || (rope->page_table != nullptr && rope->P > 0 && rope->page_size > 0)) &&
                    N >= (rope->Hq + (rope->pool != nullptr ? 2 * rope->Hkv : 0)) * rope->D && N % ROWS == 0 && ksplit == 1 &&
                    !swiglu && residual == nullptr && conv_out == nullptr && out != nullptr && out_dtype == XS_BF16),
               "gemm (few rows): the rotation behind the product needs a bfloat16 output that begins with the heads "
               "(size 32, 64 or 128) and one K slice");
    XS_REQUIRE(conv_out == nullptr ||
                   (conv_taps != nullptr && conv_state != nullptr && conv_slots != nullptr && conv_counters != nullptr &&
                    conv_k >= 2 && conv_h > 0 && conv_h % ROWS == 0 && N == 3 * conv_h && ksplit == 1 && !swiglu &&
                    residual == nullptr && out != nullptr && out_dtype == XS_BF16),
               "gemm (few rows): the convolution behind the product needs a bfloat16 output of 3 x %d columns (a multiple "
               "of 16 channels), one K slice, %d taps", conv_h, conv_k);
    XS_REQUIRE(amax_out == nullptr || (amax_keys != nullptr && amax_counter != nullptr && !swiglu && (uintptr_t)amax_keys % 8 == 0),
               "gemm (few rows): the argmax behind the product needs its keys and its counter");
    XS_REQUIRE(in_ssq == nullptr || (in_tiles > 0 && in_width > 0 && (uintptr_t)in_ssq % 16 == 0),
               "gemm (few rows): %d tiles of sums over a width of %d", in_tiles, in_width);
    XS_REQUIRE((next_x == nullptr) == (next_w == nullptr) && (next_x == nullptr || (out_ssq != nullptr && ld_next >= N)),
               "gemm (few rows): the next norm's weight, its input and the sums of squares come together");
    XS_REQUIRE(out_ssq == nullptr || residual != nullptr, "gemm (few rows): sums of squares are of the residual stream");
    XS_REQUIRE(xs_gemm_small_m_supports(M, K, ldx, ldw), "gemm (few rows): M %d, K %d, strides %lld, %lld not supported",
               M, K, (long long)ldx, (long long)ldw);
    XS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm (few rows): operands must be 16-byte aligned");
    XS_REQUIRE(N > 0 && K > 0 && ldo >= (swiglu ? N / 2 : N) && (out != nullptr || residual != nullptr),
               "gemm (few rows): bad sizes");
    XS_REQUIRE(!swiglu || (N % 16 == 0 && residual == nullptr), "gemm (few rows): the fused activation needs N %% 16 == 0");
    XS_REQUIRE(ksplit >= 1 && ksplit <= 64, "gemm (few rows): %d K slices", ksplit);
    const int tiles = ceil_div_i(N, ROWS);
    if (g_small_m_wave == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        g_small_m_wave = sms > 0 ? 4 * sms : 592;
    }
    SmallMParams p;
    p.x = (const __nv_bfloat16*)x;
    p.w = (const __nv_bfloat16*)w;
    p.bias = bias;
    p.out = out;
    p.residual = residual;
    p.partials = nullptr;
    p.counters = nullptr;
    p.M = M; p.N = N; p.K = K; p.ksplit = ksplit; p.swiglu = swiglu;
    p.wave = g_small_m_wave / ksplit;
    p.ldx = ldx; p.ldw = ldw; p.ldo = ldo;
    p.in_ssq = in_ssq; p.in_tiles = in_tiles; p.in_width = in_width; p.in_eps = in_eps;
    p.next_w = next_w; p.next_x = (__nv_bfloat16*)next_x; p.ld_next = ld_next; p.out_ssq = out_ssq;
    p.conv_taps = conv_taps; p.conv_bias = conv_bias; p.conv_state = (__nv_bfloat16*)conv_state; p.conv_slots = conv_slots;
    p.conv_out = (__nv_bfloat16*)conv_out; p.conv_counters = (unsigned int*)conv_counters; p.conv_k = conv_k; p.conv_h = conv_h;
    p.amax_keys = (unsigned long long*)amax_keys; p.amax_counter = (unsigned int*)amax_counter; p.amax_out = amax_out;
    p.rope_q = nullptr;
    if (rope != nullptr) {
        p.rope_q = (__nv_bfloat16*)rope->q_out; p.rope_pool = (__nv_bfloat16*)rope->pool; p.rope_table = rope->page_table;
        p.rope_seq = rope->seq_of_token; p.rope_pos = rope->positions; p.rope_qw = rope->q_w; p.rope_kw = rope->k_w;
        p.rope_cs = (const float2*)rope->cs; p.rope_P = rope->P; p.rope_hq = rope->Hq; p.rope_hkv = rope->Hkv;
        p.rope_d = rope->D; p.rope_page = rope->page_size; p.rope_eps = rope->eps;
    }
    if (ksplit > 1) {
        const int64_t need = xs_gemm_small_m_scratch_bytes(M, N, ksplit);
        XS_REQUIRE(scratch != nullptr && scratch_bytes >= need && (uintptr_t)scratch % 16 == 0 && scratch_bytes % 16 == 0,
                   "gemm (few rows): %lld bytes of scratch needed for %d K slices, %lld given", (long long)need, ksplit,
                   (long long)scratch_bytes);
        XS_REQUIRE((int64_t)tiles * (int64_t)sizeof(unsigned int) <= kCounterBytes, "gemm (few rows): %d row tiles", tiles);
        p.partials = (float*)scratch;
        p.counters = (unsigned int*)((char*)scratch + scratch_bytes - kCounterBytes);
    }
    // (the rotation behind the product: clusters of the D / 16 CTAs of a head; the grid is rounded up to whole clusters)
    const int per_head = rope != nullptr ? rope->D / ROWS : 1;
    const dim3 grid(ceil_div_i(tiles, per_head) * per_head, ksplit);
    // (9 to 16 rows: the unpredicated loop needs 78 registers, three CTAs an SM; with sixteen loads a round, 128 and two.
    // Measured on the whole decode step, 1.2B shape, batch 16: 1.05 ms predicated, 1.03 unpredicated, 0.99 with sixteen
    // loads, against 0.93 with the library product, which is why the default keeps this kernel to 8 rows.)
    // (the unpredicated instances load 32 bytes a lane: operands and rows on 32-byte boundaries)
    // and K slices of whole pairs of k blocks; a slice that is no multiple of 1,024 has a short last round (`ragged`)
    const bool exact = N % ROWS == 0 && K % ksplit == 0 && (K / ksplit) % 64 == 0 && (uintptr_t)x % 32 == 0 &&
                       (uintptr_t)w % 32 == 0 && ldx % 16 == 0 && ldw % 16 == 0;
    p.ragged = exact && (K / ksplit) % K_PER_CTA != 0;
    p.cluster = (g_small_m_cluster && ksplit >= 2 && ksplit <= 8) ? 1 : 0;
    // sixteen loads a round: slices that are multiples of 2,048 and at most one wave of two CTAs an SM
    const bool one_round = exact && g_small_m_one_round && (K / ksplit) % (2 * K_PER_CTA) == 0 &&
                           (int64_t)tiles * ksplit <= (g_small_m_one_round > 1 ? g_small_m_one_round : (int64_t)(g_small_m_wave / 4) * 2);
    // (the convolution behind the product: clusters of the three CTAs of a group of channels; its K is one slice)
    const dim3 cl(conv_out != nullptr ? 3 : per_head, p.cluster ? ksplit : 1, 1);
#define XS_GO(NT, TO, TAIL)                                                                                 \
    ((one_round && NT == 1) ? xs_launch_cluster(gemm_small_m_kernel<1, TO, true, 8, TAIL>, grid, dim3(WARPS * 32), 0, stream, cl, p) \
     : (exact && NT == 2 && (K / ksplit) % (2 * K_PER_CTA) == 0) ? xs_launch_cluster(gemm_small_m_kernel<2, TO, true, 8, TAIL>, grid, dim3(WARPS * 32), 0, stream, cl, p) \
     : exact ? xs_launch_cluster(gemm_small_m_kernel<NT, TO, true, UNROLL_DEFAULT, TAIL>, grid, dim3(WARPS * 32), 0, stream, cl, p)  \
             : xs_launch_cluster(gemm_small_m_kernel<NT, TO, false, UNROLL_DEFAULT, TAIL>, grid, dim3(WARPS * 32), 0, stream, cl, p))
#define XS_GO_NT(TO, TAIL) do { if (M <= 8) XS_GO(1, TO, TAIL); else XS_GO(2, TO, TAIL); } while (0)
    if (out_dtype == XS_F32 || residual != nullptr) {
        if (amax_out != nullptr) XS_GO_NT(float, 3); else XS_GO_NT(float, 0);
    } else if (out_dtype == XS_BF16) {
        if (conv_out != nullptr) XS_GO_NT(__nv_bfloat16, 1);
        else if (rope != nullptr) XS_GO_NT(__nv_bfloat16, 2);
        else if (amax_out != nullptr) XS_GO_NT(__nv_bfloat16, 3);
        else XS_GO_NT(__nv_bfloat16, 0);
    } else {
        XS_REQUIRE(false, "gemm (few rows): output type code %d", out_dtype);
    }
#undef XS_GO_NT
#undef XS_GO
    XS_LAUNCH_CHECK("gemm_small_m");
    return 0;
}

XS_API int xs_gemm_small_m_ex(const void* x, const void* w, const float* bias, void* out, float* residual,
                              int out_dtype, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int swiglu,
                              int ksplit, void* scratch, int64_t scratch_bytes, const float* in_ssq, int in_tiles,
                              int in_width, float in_eps, const float* next_w, void* next_x, int64_t ld_next,
                              float* out_ssq, const float* conv_taps, const float* conv_bias, void* conv_state,
                              const int32_t* conv_slots, void* conv_out, void* conv_counters, int conv_k, int conv_h,
                              void* amax_keys, void* amax_counter, int32_t* amax_out, cudaStream_t stream) {
    return small_m_launch(x, w, bias, out, residual, out_dtype, M, N, K, ldx, ldw, ldo, swiglu, ksplit, scratch, scratch_bytes,
                          in_ssq, in_tiles, in_width, in_eps, next_w, next_x, ld_next, out_ssq, conv_taps, conv_bias, conv_state,
                          conv_slots, conv_out, conv_counters, conv_k, conv_h, amax_keys, amax_counter, amax_out, nullptr, stream);
}

// The q/k/v product of a decode step with the per-head norm, the rotation and the cache write behind it (see XsRopeTail).
XS_API int xs_gemm_small_m_rope(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, int64_t ldx,
                                int64_t ldw, int64_t ldo, const float* in_ssq, int in_tiles, int in_width, float in_eps,
                                void* q_out, void* pool, const int32_t* page_table, int P, const int32_t* seq_of_token,
                                const int32_t* positions, const float* q_w, const float* k_w, const float* cs, int Hq,
                                int Hkv, int D, int page_size, float eps, cudaStream_t stream) {
    XsRopeTail rope;
    rope.q_out = q_out; rope.pool = pool; rope.page_table = page_table; rope.seq_of_token = seq_of_token;
    rope.positions = positions; rope.q_w = q_w; rope.k_w = k_w; rope.cs = cs; rope.P = P; rope.Hq = Hq; rope.Hkv = Hkv;
    rope.D = D; rope.page_size = page_size; rope.eps = eps;
    return small_m_launch(x, w, bias, out, nullptr, XS_BF16, M, N, K, ldx, ldw, ldo, 0, 1, nullptr, 0, in_ssq, in_tiles,
                          in_width, in_eps, nullptr, nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                          0, 0, nullptr, nullptr, nullptr, &rope, stream);
}

XS_API int xs_gemm_small_m_normed(const void* x, const void* w, const float* bias, void* out, float* residual,
                                  int out_dtype, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int swiglu,
                                  int ksplit, void* scratch, int64_t scratch_bytes, const float* in_ssq, int in_tiles,
                                  int in_width, float in_eps, const float* next_w, void* next_x, int64_t ld_next,
                                  float* out_ssq, cudaStream_t stream) {
    return xs_gemm_small_m_ex(x, w, bias, out, residual, out_dtype, M, N, K, ldx, ldw, ldo, swiglu, ksplit, scratch,
                              scratch_bytes, in_ssq, in_tiles, in_width, in_eps, next_w, next_x, ld_next, out_ssq, nullptr,
                              nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, nullptr, nullptr, stream);
}

XS_API int xs_gemm_small_m(const void* x, const void* w, const float* bias, void* out, float* residual, int out_dtype,
                           int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int swiglu, int ksplit,
                           void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    return xs_gemm_small_m_normed(x, w, bias, out, residual, out_dtype, M, N, K, ldx, ldw, ldo, swiglu, ksplit, scratch,
                                  scratch_bytes, nullptr, 0, 0, 0.0f, nullptr, nullptr, 0, nullptr, stream);
}
