// Per-head q/k RMSNorm + rotary encoding + cache write, and attention over the paged
// cache, for any head size that is a multiple of 2 up to 256, any head counts.
//
// Cache of one layer call: [pages, 2 (keys, values), kv_heads, page_size, head_dim].
// A sequence's logical page p is physical page table[seq, p]. Keys are stored normed and
// rotated, values raw (src/models/common/blocks.cpp:151-175). Query at absolute position
// pos sees key j iff j <= pos and (window == 0 or pos - j < window)
// (src/backend/cpu_ref/ops.cpp:567-571); head h reads kv head h / (heads / kv_heads)
// (ops.cpp:588). Scores, softmax and the weighted sum are float32.
#include "common.cuh"

namespace {

constexpr int kMaxHeadDim = 256;

// One warp per (token, head) over the q heads, then the k heads, then the v heads.
template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* __restrict__ qkv, int64_t ld, T* __restrict__ q_out,
                                          T* __restrict__ pool, const int32_t* __restrict__ page_table, int P,
                                          const int32_t* __restrict__ seq_of_token,
                                          const int32_t* __restrict__ positions, const float* __restrict__ q_w,
                                          const float* __restrict__ k_w, const float2* __restrict__ rope, int Tn,
                                          int Hq, int Hkv, int D, int page_size, float eps, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int heads_total = Hq + (write_kv ? 2 * Hkv : 0);
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)Tn * heads_total) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(item / heads_total);
    const int hh = (int)(item % heads_total);
    const int half = D >> 1;
    const int pos = positions[t];
    const T* src = qkv + (int64_t)t * ld + (int64_t)hh * D;   // q heads, k heads, v heads are consecutive

    T* dst;
    const float* w;
    bool rotate;
    if (hh < Hq) {
        dst = q_out + ((int64_t)t * Hq + hh) * D;
        w = q_w;
        rotate = true;
    } else {
        const int kvh = (hh - Hq) % Hkv;
        const int which = (hh - Hq) / Hkv;   // 0 keys, 1 values
        const int seq = seq_of_token[t];
        const int page = page_table[(int64_t)seq * P + pos / page_size];
        dst = pool + ((((int64_t)page * 2 + which) * Hkv + kvh) * page_size + pos % page_size) * D;
        w = which == 0 ? k_w : nullptr;
        rotate = which == 0;
    }
    if (!rotate) {   // values: a plain copy
        for (int d = lane; d < D; d += 32) dst[d] = src[d];
        return;
    }
    // pair i couples channels i and i + D/2
    float a[kMaxHeadDim / 64], b[kMaxHeadDim / 64];
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < kMaxHeadDim / 64; ++u) {
        const int i = lane + 32 * u;
        if (i < half) {
            a[u] = to_f32(src[i]);
            b[u] = to_f32(src[i + half]);
            ss += a[u] * a[u] + b[u] * b[u];
        }
    }
    float inv = 1.0f;
    if (w != nullptr) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)D + eps);
    }
#pragma unroll
    for (int u = 0; u < kMaxHeadDim / 64; ++u) {
        const int i = lane + 32 * u;
        if (i < half) {
            float x1 = a[u], x2 = b[u];
            if (w != nullptr) {
                x1 = x1 * inv * w[i];
                x2 = x2 * inv * w[i + half];
            }
            if (rope != nullptr) {
                const float2 cs = rope[(int64_t)pos * half + i];
                const float r1 = x1 * cs.x - x2 * cs.y;
                const float r2 = x2 * cs.x + x1 * cs.y;
                x1 = r1;
                x2 = r2;
            }
            dst[i] = from_f32<T>(x1);
            dst[i + half] = from_f32<T>(x2);
        }
    }
}

// bfloat16, head sizes 16, 32, 64, 128, 256: a thread owns 8 neighbouring channels (one 16-byte load and
// store), the D / 8 threads of a head are neighbours in a warp; the sum of squares and the partner channels
// (i and i + D / 2 sit D / 16 lanes apart) travel by shuffles.
template <int D>
__global__ void __launch_bounds__(256) qk_norm_rope_store_vec_kernel(
    const __nv_bfloat16* __restrict__ qkv, int64_t ld, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ pool,
    const int32_t* __restrict__ page_table, int P, const int32_t* __restrict__ seq_of_token,
    const int32_t* __restrict__ positions, const float* __restrict__ q_w, const float* __restrict__ k_w,
    const float2* __restrict__ rope, int Tn, int Hq, int Hkv, int page_size, float eps, int write_kv) {
    constexpr int G = D / 8;        // threads of a head
    constexpr int half = D / 2;
    pdl_launch_dependents();
    // Positions, page numbers, norm weights and the rotation table are not written by the kernel before this one
    // (the q/k/v product): they are read before waiting for it, and only the product's output after.
    const int heads_total = Hq + (write_kv ? 2 * Hkv : 0);
    const int64_t thread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = thread / G;
    const int part = (int)(thread % G);
    const bool live = item < (int64_t)Tn * heads_total;     // dead threads still take part in the shuffles
    const int t = live ? (int)(item / heads_total) : 0;
    const int hh = live ? (int)(item % heads_total) : 0;
    const int pos = positions[t];
    const int c0 = part * 8;

    __nv_bfloat16* dst;
    const float* w;
    bool rotate;
    if (hh < Hq) {
        dst = q_out + ((int64_t)t * Hq + hh) * D + c0;
        w = q_w;
        rotate = true;
    } else {
        const int kvh = (hh - Hq) % Hkv;
        const int which = (hh - Hq) / Hkv;
        const int seq = seq_of_token[t];
        const int page = page_table[(int64_t)seq * P + pos / page_size];
        dst = pool + ((((int64_t)page * 2 + which) * Hkv + kvh) * page_size + pos % page_size) * D + c0;
        w = which == 0 ? k_w : nullptr;
        rotate = which == 0;
    }
    float wv[8];
    if (rotate && w != nullptr) {
        const float4 w0 = *reinterpret_cast<const float4*>(w + c0), w1 = *reinterpret_cast<const float4*>(w + c0 + 4);
        wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w;
        wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
    }
    const bool low = c0 < half;
    float2 cs[8];
    if (rotate && rope != nullptr) {
        const float2* at = rope + (int64_t)pos * half + (low ? c0 : c0 - half);
#pragma unroll
        for (int j = 0; j < 8; ++j) cs[j] = at[j];
    }
    pdl_wait();
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = *reinterpret_cast<const uint4*>(qkv + (int64_t)t * ld + (int64_t)hh * D + c0);
    float x[8];
    {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            x[2 * j] = f.x;
            x[2 * j + 1] = f.y;
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (rotate && w != nullptr) {
        const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = x[j] * inv * wv[j];
    }
    // the partner's 8 channels: i + D/2 for the lower half, i - D/2 for the upper half
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = G > 1 ? __shfl_xor_sync(0xffffffffu, x[j], G / 2) : 0.0f;
    if (rotate && rope != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 a = cs[j];
            // low: x1 cos - x2 sin with x1 = x, x2 = y; high: x2 cos + x1 sin with x2 = x, x1 = y
            x[j] = low ? x[j] * a.x - y[j] * a.y : x[j] * a.x + y[j] * a.y;
        }
    }
    if (!live) return;
    if (rotate) {
        uint4 o;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
        *reinterpret_cast<uint4*>(dst) = o;
    } else {
        *reinterpret_cast<uint4*>(dst) = raw;     // values: a plain copy
    }
}

// One warp per (token, q head). Scores with lanes over keys, weighted sum with lanes over channels.
template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ pool,
                                         const int32_t* __restrict__ page_table, int P,
                                         const int32_t* __restrict__ seq_of_token,
                                         const int32_t* __restrict__ positions, const T* __restrict__ gate,
                                         int64_t ld_gate, T* __restrict__ out, int Tn, int Hq, int Hkv, int D,
                                         int page_size, float scale, int window) {
    extern __shared__ float q_sm[];   // [warps][D]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (int64_t)Tn * Hq) return;
    const int t = (int)(item / Hq), h = (int)(item % Hq);
    const int kvh = h / (Hq / Hkv);
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int32_t* table = page_table + (int64_t)seq * P;
    float* qs = q_sm + warp * D;
    const T* qrow = q + ((int64_t)t * Hq + h) * D;
    for (int d = lane; d < D; d += 32) qs[d] = to_f32(qrow[d]) * scale;
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int u = 0; u < kMaxHeadDim / 32; ++u) acc[u] = 0.0f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = table[j / page_size];
            const T* kr = pool + ((((int64_t)page * 2 + 0) * Hkv + kvh) * page_size + j % page_size) * D;
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = j <= pos ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);   // 0 on the first block (m = -inf)
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int u = 0; u < kMaxHeadDim / 32; ++u) acc[u] *= corr;
        const int cnt = min(32, pos - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int jk = j0 + jj;
            const int page = table[jk / page_size];
            const T* vr = pool + ((((int64_t)page * 2 + 1) * Hkv + kvh) * page_size + jk % page_size) * D;
#pragma unroll
            for (int u = 0; u < kMaxHeadDim / 32; ++u) {
                const int d = lane + 32 * u;
                if (d < D) acc[u] = fmaf(pj, to_f32(vr[d]), acc[u]);
            }
        }
    }
    float g = 1.0f;
    if (gate != nullptr) {
        const float z = to_f32(gate[(int64_t)t * ld_gate + h]);
        g = 1.0f / (1.0f + expf(-z));
    }
    const float norm = g / l;
    T* orow = out + ((int64_t)t * Hq + h) * D;
#pragma unroll
    for (int u = 0; u < kMaxHeadDim / 32; ++u) {
        const int d = lane + 32 * u;
        if (d < D) orow[d] = from_f32<T>(acc[u] * norm);
    }
}

}  // namespace

XS_API int xs_qk_norm_rope_store(const void* qkv, int64_t ld, void* q_out, void* pool, const int32_t* page_table,
                                 int P, const int32_t* seq_of_token, const int32_t* positions, const float* q_w,
                                 const float* k_w, const float* rope, int T, int Hq, int Hkv, int D, int page_size,
                                 float eps, int write_kv, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(D > 0 && D % 2 == 0 && D <= kMaxHeadDim, "qk_norm_rope: head size %d (even, at most %d)", D, kMaxHeadDim);
    XS_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "qk_norm_rope: %d heads over %d kv heads", Hq, Hkv);
    XS_REQUIRE(!write_kv || (pool != nullptr && page_table != nullptr && P > 0), "qk_norm_rope: no cache to write to");
    const int64_t items = (int64_t)T * (Hq + (write_kv ? 2 * Hkv : 0));
    // bfloat16 with 16-byte rows everywhere and a head size whose halves sit a power of two of lanes apart
    const bool vec = dtype == XS_BF16 && (D == 16 || D == 32 || D == 64 || D == 128 || D == 256) && ld % 8 == 0 &&
                     (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (!write_kv || (uintptr_t)pool % 16 == 0) &&
                     (q_w == nullptr || (uintptr_t)q_w % 16 == 0) && (k_w == nullptr || (uintptr_t)k_w % 16 == 0);
    if (vec) {
        const int vblocks = ceil_div_i(items * (D / 8), 256);
#define XS_ROPE_VEC(DD)                                                                                            \
    xs_launch(qk_norm_rope_store_vec_kernel<DD>, dim3(vblocks), dim3(256), 0, stream, (const __nv_bfloat16*)qkv, ld, \
              (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, page_table, P, seq_of_token, positions, q_w, k_w,        \
              (const float2*)rope, T, Hq, Hkv, page_size, eps, write_kv)
        switch (D) {
            case 16: XS_ROPE_VEC(16); break;
            case 32: XS_ROPE_VEC(32); break;
            case 64: XS_ROPE_VEC(64); break;
            case 128: XS_ROPE_VEC(128); break;
            default: XS_ROPE_VEC(256); break;
        }
#undef XS_ROPE_VEC
        XS_LAUNCH_CHECK("qk_norm_rope_store");
        return 0;
    }
    const int blocks = ceil_div_i(items, 4);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(qk_norm_rope_store_kernel<TT>, dim3(blocks), dim3(128), 0, stream,
                          (const TT*)qkv, ld, (TT*)q_out, (TT*)pool, page_table, P, seq_of_token, positions, q_w,
                          k_w, (const float2*)rope, T, Hq, Hkv, D, page_size, eps, write_kv));
    XS_LAUNCH_CHECK("qk_norm_rope_store");
    return 0;
}

XS_API int xs_attention_generic(const void* q, const void* pool, const int32_t* page_table, int P,
                                const int32_t* seq_of_token, const int32_t* positions, const void* gate,
                                int64_t ld_gate, void* out, int T, int Hq, int Hkv, int D, int page_size,
                                float scale, int window, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(D > 0 && D % 2 == 0 && D <= kMaxHeadDim, "attention: head size %d (even, at most %d)", D, kMaxHeadDim);
    XS_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: %d heads over %d kv heads", Hq, Hkv);
    XS_REQUIRE(window >= 0 && page_size > 0 && P > 0, "attention: window %d, page size %d, %d pages", window, page_size, P);
    const int warps = 4;
    const int blocks = ceil_div_i((int64_t)T * Hq, warps);
    const size_t smem = (size_t)warps * D * sizeof(float);
    XS_DISPATCH_DTYPE(dtype, TT,
                      attention_generic_kernel<TT><<<blocks, warps * 32, smem, stream>>>(
                          (const TT*)q, (const TT*)pool, page_table, P, seq_of_token, positions, (const TT*)gate,
                          ld_gate, (TT*)out, T, Hq, Hkv, D, page_size, scale, window));
    XS_LAUNCH_CHECK("attention_generic");
    return 0;
}
