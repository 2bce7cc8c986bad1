// out[M, N] = x[M, K] . w[N, K]^T (+ bias[N]), any sizes, float32 accumulation.
//
// The plain matrix product of the float32 path and the fallback of the bfloat16 path:
// CUDA-core FMAs only, no tensor cores and no reduced-precision mode. Each output
// element sums its K products in an order that depends on K alone (32 at a time into
// a partial, partials added in ascending k), so a row's result is the same bit for
// bit whatever the other rows of the batch are. The reference's cpu-ref sums in
// float64 (src/backend/cpu_ref/ops.cpp:96-108, 157-199); weights are [out, in]
// (src/graph/graph.h:12,46).
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 32;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const float* __restrict__ bias,
                    TO* __restrict__ out, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo) {
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[TK][TN + 1];
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 32 k of each operand; thread -> (row = idx / 32, k = idx % 32), 8 passes
        for (int idx = threadIdx.x; idx < TM * TK; idx += 256) {
            const int r = idx >> 5, k = idx & 31;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            xs[k][r] = (gm < M && gk < K) ? to_f32(x[(int64_t)gm * ldx + gk]) : 0.0f;
            ws[k][r] = (gn < N && gk < K) ? to_f32(w[(int64_t)gn * ldw + gk]) : 0.0f;
        }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.0f;
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += bias[gn];
            out[(int64_t)gm * ldo + gn] = from_f32<TO>(v);
        }
    }
}

}  // namespace

// x and w share one element type; out is float32 or that type.
XS_API int xs_gemm_generic(const void* x, const void* w, const float* bias, void* out, int in_dtype, int out_dtype,
                           int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    XS_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: sizes %d x %d x %d", M, N, K);
    XS_REQUIRE(ldx >= K && ldw >= K && ldo >= N, "gemm: a row stride is shorter than its row");
    const dim3 grid(ceil_div_i(N, TN), ceil_div_i(M, TM));
    XS_REQUIRE(grid.y <= 65535, "gemm: %d rows exceed the grid limit", M);
    if (in_dtype == XS_F32 && out_dtype == XS_F32) {
        gemm_generic_kernel<float, float, float><<<grid, 256, 0, stream>>>((const float*)x, (const float*)w, bias,
                                                                          (float*)out, M, N, K, ldx, ldw, ldo);
    } else if (in_dtype == XS_BF16 && out_dtype == XS_F32) {
        gemm_generic_kernel<__nv_bfloat16, __nv_bfloat16, float><<<grid, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, (float*)out, M, N, K, ldx, ldw, ldo);
    } else if (in_dtype == XS_BF16 && out_dtype == XS_BF16) {
        gemm_generic_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo);
    } else {
        XS_REQUIRE(false, "gemm: element types in %d, out %d are not supported", in_dtype, out_dtype);
    }
    XS_LAUNCH_CHECK("gemm_generic");
    return 0;
}
