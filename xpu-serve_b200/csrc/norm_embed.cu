// Embedding gather, fused residual-add + RMSNorm, SwiGLU activation, error state.
//
// RMSNorm(x, w, eps) = x * (mean(x^2) + eps)^(-1/2) * w over the last dimension, no +1
// offset, all in float32 (reference: src/graph/graph.h:57, kernel
// src/backend/sycl/sycl_kernels.cpp:1543-1559). The residual stream is float32 in every
// precision mode; a branch's output joins it here.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void xs_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

XS_API const char* xs_last_error() { return g_error; }

XS_API int xs_abi_version() { return 5; }

int g_xs_pdl = 1;
// 1: kernels of a step may overlap their start with the previous kernel's end (programmatic
// dependent launch); 0: plain stream order. Returns the previous setting.
XS_API int xs_set_pdl(int on) {
    const int old = g_xs_pdl;
    g_xs_pdl = on ? 1 : 0;
    return old;
}

// ------------------------------------------------------------------ embedding
// h[t, :] = table[ids[t], :] * scale as float32 (LFM3: scale 1, src/models/lfm3/lfm3_decoder.cpp:50).
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int32_t* __restrict__ ids,
                             float* __restrict__ h, int T, int H, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const TW* row = table + (int64_t)ids[t] * H;
    float* out = h + (int64_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[c] = to_f32(row[c]) * scale;
}

// logits = cap * tanh(logits / cap), in place: a soft limit that some architectures put on their logits.
__global__ void logit_cap_kernel(float* __restrict__ logits, int64_t n, float cap, float inv_cap) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        logits[i] = cap * tanhf(logits[i] * inv_cap);
}

XS_API int xs_embed(const void* table, int table_dtype, const int32_t* ids, float* h, int T, int H, float scale,
                    cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && H > 0, "embed: %d tokens of width %d", T, H);
    XS_DISPATCH_DTYPE(table_dtype, TW,
                      xs_launch(embed_kernel<TW>, dim3(T), dim3(256), 0, stream, (const TW*)table, ids, h, T, H, scale));
    XS_LAUNCH_CHECK("embed");
    return 0;
}

XS_API int xs_logit_cap(float* logits, int64_t n, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    XS_REQUIRE(n > 0 && cap > 0.0f, "logit cap: %lld values, cap %g", (long long)n, (double)cap);
    const int blocks = (int)(n / 1024 < 1 ? 1 : (n / 1024 > 1184 ? 1184 : n / 1024));
    xs_launch(logit_cap_kernel, dim3(blocks), dim3(256), 0, stream, logits, n, cap, 1.0f / cap);
    XS_LAUNCH_CHECK("logit_cap");
    return 0;
}

// ------------------------------------------------------- add + RMSNorm (fused)
// For each output row i (source row r = rows ? rows[i] : i):
//   v = h[r]                                   float32
//   if m:      b = m[r];  if post_w: b = RMSNorm(b, post_w, eps_post)
//              v = v + b;  h[r] = v            the residual sum stays float32
//   if w:      y[i] = RMSNorm(v, w, eps)       written in y's element type
// One block per row; the row lives in shared memory between the passes.
template <typename TM, typename TY>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TM* __restrict__ m,
                                   const float* __restrict__ post_w, const float* __restrict__ w,
                                   TY* __restrict__ y, const int32_t* __restrict__ rows, int H, float eps_post, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* hr = h + r * H;
    float ss = 0.0f;
    if (m != nullptr) {
        const TM* mr = m + r * H;
        if (post_w != nullptr) {
            float bs = 0.0f;
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float b = to_f32(mr[c]);
                row[c] = b;
                bs += b * b;
            }
            bs = block_sum(bs, scratch);
            const float inv = 1.0f / sqrtf(bs / (float)H + eps_post);
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float v = hr[c] + row[c] * inv * post_w[c];
                row[c] = v;
                hr[c] = v;
                ss += v * v;
            }
        } else {
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float v = hr[c] + to_f32(mr[c]);
                row[c] = v;
                hr[c] = v;
                ss += v * v;
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = hr[c];
            row[c] = v;
            ss += v * v;
        }
    }
    if (w == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TY* yr = y + (int64_t)i * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) yr[c] = from_f32<TY>(row[c] * inv * w[c]);
}


// The same operation for widths that are a multiple of 4 and at most 16 * 1024: each thread keeps
// up to four float4 of the row in registers, so the row is read once and every pass after the
// first runs on registers.
template <typename TM>
__device__ __forceinline__ float4 load4(const TM* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TM, typename TY, int NV>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TM* __restrict__ m,
                                       const float* __restrict__ post_w, const float* __restrict__ w,
                                       TY* __restrict__ y, const int32_t* __restrict__ rows, int H, float eps_post,
                                       float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* hr = h + r * H;
    const int chunks = H >> 2;
    float4 v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = c < chunks ? load4<float>(hr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (m != nullptr) {
        const TM* mr = m + r * H;
        float4 b[NV];
        float bs = 0.0f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            b[k] = c < chunks ? load4<TM>(mr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
            bs += b[k].x * b[k].x + b[k].y * b[k].y + b[k].z * b[k].z + b[k].w * b[k].w;
        }
        float inv = 1.0f;
        if (post_w != nullptr) {
            bs = block_sum(bs, scratch);
            inv = 1.0f / sqrtf(bs / (float)H + eps_post);
        }
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c >= chunks) continue;
            float4 pw = make_float4(1.f, 1.f, 1.f, 1.f);
            if (post_w != nullptr) pw = load4<float>(post_w + 4 * c);
            if (post_w != nullptr) {
                v[k].x += b[k].x * inv * pw.x;
                v[k].y += b[k].y * inv * pw.y;
                v[k].z += b[k].z * inv * pw.z;
                v[k].w += b[k].w * inv * pw.w;
            } else {
                v[k].x += b[k].x;
                v[k].y += b[k].y;
                v[k].z += b[k].z;
                v[k].w += b[k].w;
            }
            store4(hr + 4 * c, v[k]);
        }
    }
    if (w == nullptr) return;
#pragma unroll
    for (int k = 0; k < NV; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TY* yr = y + (int64_t)i * H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c >= chunks) continue;
        const float4 ww = load4<float>(w + 4 * c);
        store4(yr + 4 * c, make_float4(v[k].x * inv * ww.x, v[k].y * inv * ww.y, v[k].z * inv * ww.z, v[k].w * inv * ww.w));
    }
}

XS_API int xs_add_rmsnorm(float* h, const void* m, int m_dtype, const float* post_w, const float* w, void* y,
                          int y_dtype, const int32_t* rows, int n_rows, int H, float eps_post, float eps,
                          cudaStream_t stream) {
    if (n_rows == 0) return 0;
    XS_REQUIRE(n_rows > 0 && H > 0, "add_rmsnorm: %d rows of width %d", n_rows, H);
    XS_REQUIRE((size_t)H * 4 <= 200 * 1024, "add_rmsnorm: width %d does not fit shared memory (limit 51200)", H);
    XS_REQUIRE(w == nullptr || y != nullptr, "add_rmsnorm: a norm weight without an output");
    const bool aligned = H % 4 == 0 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)m % 16 == 0) && ((uintptr_t)y % 16 == 0) &&
                         ((uintptr_t)w % 16 == 0) && ((uintptr_t)post_w % 16 == 0);
    if (aligned && H <= 16 * 1024) {
        const int chunks = H / 4;
        const int threads = chunks <= 128 ? 128 : chunks <= 1024 ? 256 : chunks <= 2048 ? 512 : 1024;
        const int nv = (chunks + threads - 1) / threads;
#define XS_VEC(TM, TY, NV)                                                                                          \
    xs_launch(add_rmsnorm_vec_kernel<TM, TY, NV>, dim3(n_rows), dim3(threads), 0, stream, h, (const TM*)m, post_w, \
              w, (TY*)y, rows, H, eps_post, eps)
#define XS_VEC_NV(TM, TY)                       \
    do {                                        \
        if (nv <= 1) XS_VEC(TM, TY, 1);         \
        else if (nv == 2) XS_VEC(TM, TY, 2);    \
        else XS_VEC(TM, TY, 4);                 \
    } while (0)
        XS_DISPATCH_DTYPE(m_dtype, TM, XS_DISPATCH_DTYPE(y_dtype, TY, XS_VEC_NV(TM, TY)));
#undef XS_VEC_NV
#undef XS_VEC
        XS_LAUNCH_CHECK("add_rmsnorm");
        return 0;
    }
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = H >= 2048 ? 512 : 256;
#define XS_GO(TM, TY)                                                                                    \
    do {                                                                                                 \
        if (smem > 48 * 1024)                                                                            \
            cudaFuncSetAttribute(add_rmsnorm_kernel<TM, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                             \
        xs_launch(add_rmsnorm_kernel<TM, TY>, dim3(n_rows), dim3(threads), smem, stream, h, (const TM*)m, \
                  post_w, w, (TY*)y, rows, H, eps_post, eps);                                            \
    } while (0)
    XS_DISPATCH_DTYPE(m_dtype, TM, XS_DISPATCH_DTYPE(y_dtype, TY, XS_GO(TM, TY)));
#undef XS_GO
    XS_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

// ----------------------------------------------------------------- SwiGLU act
// out[t, f] = silu(gate[t, f]) * up[t, f], silu(z) = z / (1 + exp(-z))
// (src/models/common/blocks.cpp:23-27; src/backend/cpu_ref/ops.cpp:242-247).
// Layout of a gate/up row: interleave 0: [F gate | F up]; interleave 8: blocks of 16 columns,
// 8 gate then the 8 up of the same f (how the stacked weight is ordered for the fused epilogue
// of the few-row product).
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int F, int64_t ld,
                                int interleave) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F;
        const int f = (int)(i - t * F);
        const int64_t gi = interleave ? (int64_t)(f / interleave) * 2 * interleave + f % interleave : f;
        const int64_t ui = interleave ? gi + interleave : (int64_t)F + f;
        out[i] = from_f32<T>(silu_f(to_f32(gu[t * ld + gi])) * to_f32(gu[t * ld + ui]));
    }
}

// 8 outputs a thread, 16-byte loads and stores; F a multiple of 8, rows 16-byte aligned.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int64_t total8, int F8, int64_t ld, int interleave) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F8;
        const int j = (int)(i - t * F8);
        const __nv_bfloat16* row = gu + t * ld;
        const uint4 g = *reinterpret_cast<const uint4*>(row + (interleave ? 16 * j : 8 * j));
        const uint4 u = *reinterpret_cast<const uint4*>(row + (interleave ? 16 * j + 8 : 8 * (int64_t)F8 + 8 * j));
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
            op[k] = __floats2bfloat162_rn(silu_f(gf.x) * uf.x, silu_f(gf.y) * uf.y);
        }
        *reinterpret_cast<uint4*>(out + t * 8 * (int64_t)F8 + 8 * j) = o;
    }
}

XS_API int xs_silu_mul(const void* gu, void* out, int dtype, int T, int F, int64_t ld, int interleave,
                       cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && F > 0 && ld >= 2 * (int64_t)F, "silu_mul: %d rows, %d columns, stride %lld", T, F, (long long)ld);
    XS_REQUIRE(interleave == 0 || (interleave == 8 && F % 8 == 0), "silu_mul: interleave %d with %d columns", interleave, F);
    if (dtype == XS_BF16 && F % 8 == 0 && ld % 8 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const int64_t total8 = (int64_t)T * (F / 8);
        const int blocks = (int)((total8 + 255) / 256 < 148 * 32 ? (total8 + 255) / 256 : 148 * 32);
        xs_launch(silu_mul_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu,
                  (__nv_bfloat16*)out, total8, F / 8, ld, interleave);
        XS_LAUNCH_CHECK("silu_mul");
        return 0;
    }
    const int64_t total = (int64_t)T * F;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(silu_mul_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (const TT*)gu, (TT*)out, total, F, ld, interleave));
    XS_LAUNCH_CHECK("silu_mul");
    return 0;
}

// ------------------------------------------------------------ zero state rows
// state[slots[i], :] = 0 for a freshly opened sequence.
__global__ void zero_rows_kernel(uint8_t* __restrict__ base, const int32_t* __restrict__ slots, int64_t row_bytes) {
    uint8_t* row = base + (int64_t)slots[blockIdx.x] * row_bytes;
    for (int64_t i = threadIdx.x; i < row_bytes; i += blockDim.x) row[i] = 0;
}

XS_API int xs_zero_rows(void* base, const int32_t* slots, int n, int64_t row_bytes, cudaStream_t stream) {
    if (n == 0 || row_bytes == 0) return 0;
    zero_rows_kernel<<<n, 256, 0, stream>>>((uint8_t*)base, slots, row_bytes);
    XS_LAUNCH_CHECK("zero_rows");
    return 0;
}
