// out[M, N] = x[M, K] . w[N, K]^T for few rows (M <= 16): the decode-time matrix product.
//
// The weight is read exactly once, straight from HBM into registers with 16-byte loads, and
// never staged: with M this small the product is bound by weight bandwidth. A CTA of 8 warps
// owns 16 weight rows; its warps take the 32-wide k blocks in turn (warp w: blocks w, w+8, ...),
// multiply on tensor cores (mma.sync m16n8k16: weight rows on the M side, the batch on the N
// side) and their partial sums are added in shared memory in warp order, so the result does
// not depend on timing. A lane's 16 bytes are 8 consecutive k of one row; the same
// assignment of k to fragment slots is used for the weight and for x, which is all a
// contraction needs. The reference has the same split: its own `gemv_t` up to 8 rows, a
// library GEMM above (src/backend/sycl/sycl_kernels.cpp:630-714, sycl_kernels.h:280).
//
// Optional epilogue: bias[N] added; `residual` (float32 [M, N]) += result instead of storing
// (the branch output joining the residual stream when no norm stands between).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int ROWS = 16;   // weight rows per CTA

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

template <int NT, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                    const float* __restrict__ bias, TO* __restrict__ out, float* __restrict__ residual, int M, int N,
                    int K, int64_t ldx, int64_t ldw, int64_t ldo, int swiglu) {
    __shared__ float red[WARPS][ROWS][8 * NT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int ra = min(n0 + g, N - 1), rb = min(n0 + g + 8, N - 1);   // clamped: out-of-range rows are not stored
    const __nv_bfloat16* wa_p = w + (int64_t)ra * ldw + q * 8;
    const __nv_bfloat16* wb_p = w + (int64_t)rb * ldw + q * 8;
    const __nv_bfloat16* x_p[NT];
    bool x_ok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        x_ok[t] = t * 8 + g < M;
        x_p[t] = x + (int64_t)(x_ok[t] ? t * 8 + g : 0) * ldx + q * 8;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;

    const int k_blocks = (K + 31) / 32;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    constexpr int UNROLL = 4;
    for (int kb = warp; kb < k_blocks; kb += WARPS * UNROLL) {
        uint4 wa[UNROLL], wb[UNROLL], xv[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k0 = (kb + u * WARPS) * 32;
            const bool in = k0 + q * 8 < K;      // K is a multiple of 8: a lane's 8 elements are all in or all out
            wa[u] = in ? ld_stream(wa_p + k0) : zero;
            wb[u] = in ? ld_stream(wb_p + k0) : zero;
#pragma unroll
            for (int t = 0; t < NT; ++t)
                xv[u][t] = (in && x_ok[t]) ? *reinterpret_cast<const uint4*>(x_p[t] + k0) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                mma_bf16_16816(acc[t], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv[u][t].x, xv[u][t].y);
                mma_bf16_16816(acc[t], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv[u][t].z, xv[u][t].w);
            }
        }
    }
    // c0, c1: (weight row g, batch q * 2 + {0, 1}); c2, c3: weight row g + 8
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        red[warp][g][t * 8 + q * 2] = acc[t][0];
        red[warp][g][t * 8 + q * 2 + 1] = acc[t][1];
        red[warp][g + 8][t * 8 + q * 2] = acc[t][2];
        red[warp][g + 8][t * 8 + q * 2 + 1] = acc[t][3];
    }
    __syncthreads();
    if (swiglu) {
        // The weight's rows come in blocks of 16: 8 gate rows, then the 8 up rows of the same outputs.
        // out[m, n0 / 2 + r] = silu(gate_r) * up_r: the activation is never written unfused.
        for (int i = threadIdx.x; i < 8 * 8 * NT; i += WARPS * 32) {
            const int r = i % 8, m = i / 8;
            if (m >= M || n0 + 8 + r >= N) continue;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; ++wv) {
                gate += red[wv][r][m];
                up += red[wv][r + 8][m];
            }
            if (bias != nullptr) {
                gate += bias[n0 + r];
                up += bias[n0 + 8 + r];
            }
            out[(int64_t)m * ldo + (n0 >> 1) + r] = from_f32<TO>(gate / (1.0f + expf(-gate)) * up);
        }
        return;
    }
    for (int i = threadIdx.x; i < ROWS * 8 * NT; i += WARPS * 32) {
        const int r = i % ROWS, m = i / ROWS;       // neighbouring threads write neighbouring columns of out
        const int n = n0 + r;
        if (m >= M || n >= N) continue;
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) v += red[wv][r][m];
        if (bias != nullptr) v += bias[n];
        if (residual != nullptr) {
            residual[(int64_t)m * ldo + n] += v;
        } else {
            out[(int64_t)m * ldo + n] = from_f32<TO>(v);
        }
    }
}

}  // namespace

XS_API int xs_gemm_small_m_supports(int M, int K, int64_t ldx, int64_t ldw) {
    return M >= 1 && M <= 16 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

// x, w bfloat16; out bfloat16 or float32 (out_dtype), or residual += when `residual` is given (float32, stride ldo).
// swiglu != 0: w holds blocks of 8 gate rows and 8 up rows; out is [M, N / 2] = silu(gate) * up.
XS_API int xs_gemm_small_m(const void* x, const void* w, const float* bias, void* out, float* residual, int out_dtype,
                           int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int swiglu,
                           cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    XS_REQUIRE(xs_gemm_small_m_supports(M, K, ldx, ldw), "gemm (few rows): M %d, K %d, strides %lld, %lld not supported",
               M, K, (long long)ldx, (long long)ldw);
    XS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm (few rows): operands must be 16-byte aligned");
    XS_REQUIRE(N > 0 && K > 0 && ldo >= (swiglu ? N / 2 : N) && (out != nullptr || residual != nullptr),
               "gemm (few rows): bad sizes");
    XS_REQUIRE(!swiglu || (N % 16 == 0 && residual == nullptr), "gemm (few rows): the fused activation needs N %% 16 == 0");
    const int blocks = ceil_div_i(N, ROWS);
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
#define XS_GO(NT, TO) gemm_small_m_kernel<NT, TO><<<blocks, WARPS * 32, 0, stream>>>(xp, wp, bias, (TO*)out, residual, M, N, K, ldx, ldw, ldo, swiglu)
    if (out_dtype == XS_F32 || residual != nullptr) {
        if (M <= 8) XS_GO(1, float); else XS_GO(2, float);
    } else if (out_dtype == XS_BF16) {
        if (M <= 8) XS_GO(1, __nv_bfloat16); else XS_GO(2, __nv_bfloat16);
    } else {
        XS_REQUIRE(false, "gemm (few rows): output type code %d", out_dtype);
    }
#undef XS_GO
    XS_LAUNCH_CHECK("gemm_small_m");
    return 0;
}
