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

XS_API int xs_abi_version() { return 3; }

// ------------------------------------------------------------------ embedding
// h[t, :] = table[ids[t], :] as float32 (no scaling: src/models/lfm3/lfm3_decoder.cpp:50).
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int32_t* __restrict__ ids,
                             float* __restrict__ h, int T, int H) {
    const int t = blockIdx.x;
    const TW* row = table + (int64_t)ids[t] * H;
    float* out = h + (int64_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[c] = to_f32(row[c]);
}

XS_API int xs_embed(const void* table, int table_dtype, const int32_t* ids, float* h, int T, int H,
                    cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && H > 0, "embed: %d tokens of width %d", T, H);
    XS_DISPATCH_DTYPE(table_dtype, TW,
                      embed_kernel<TW><<<T, 256, 0, stream>>>((const TW*)table, ids, h, T, H));
    XS_LAUNCH_CHECK("embed");
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

XS_API int xs_add_rmsnorm(float* h, const void* m, int m_dtype, const float* post_w, const float* w, void* y,
                          int y_dtype, const int32_t* rows, int n_rows, int H, float eps_post, float eps,
                          cudaStream_t stream) {
    if (n_rows == 0) return 0;
    XS_REQUIRE(n_rows > 0 && H > 0, "add_rmsnorm: %d rows of width %d", n_rows, H);
    XS_REQUIRE((size_t)H * 4 <= 200 * 1024, "add_rmsnorm: width %d does not fit shared memory (limit 51200)", H);
    XS_REQUIRE(w == nullptr || y != nullptr, "add_rmsnorm: a norm weight without an output");
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = H >= 2048 ? 512 : 256;
#define XS_GO(TM, TY)                                                                                    \
    do {                                                                                                 \
        if (smem > 48 * 1024)                                                                            \
            cudaFuncSetAttribute(add_rmsnorm_kernel<TM, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                             \
        add_rmsnorm_kernel<TM, TY><<<n_rows, threads, smem, stream>>>(h, (const TM*)m, post_w, w, (TY*)y, \
                                                                      rows, H, eps_post, eps);           \
    } while (0)
    XS_DISPATCH_DTYPE(m_dtype, TM, XS_DISPATCH_DTYPE(y_dtype, TY, XS_GO(TM, TY)));
#undef XS_GO
    XS_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

// ----------------------------------------------------------------- SwiGLU act
// out[t, f] = silu(gu[t, f]) * gu[t, F + f], silu(z) = z / (1 + exp(-z))
// (src/models/common/blocks.cpp:23-27; src/backend/cpu_ref/ops.cpp:242-247).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int F, int64_t ld) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F;
        const int f = (int)(i - t * F);
        const float g = to_f32(gu[t * ld + f]);
        const float u = to_f32(gu[t * ld + F + f]);
        out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

XS_API int xs_silu_mul(const void* gu, void* out, int dtype, int T, int F, int64_t ld, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && F > 0 && ld >= 2 * (int64_t)F, "silu_mul: %d rows, %d columns, stride %lld", T, F, (long long)ld);
    const int64_t total = (int64_t)T * F;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT, silu_mul_kernel<TT><<<blocks, 256, 0, stream>>>((const TT*)gu, (TT*)out, total, F, ld));
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
