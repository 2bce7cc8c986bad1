// Gated causal depthwise convolution over a ragged batch, with each sequence's own state.
//
// Input bcx[t] = [B | C | X] (3 * H wide), g = B * X. With x' = [state (K-1 rows); g of
// this step's tokens], conv[t, c] = sum_j w[c, j] * x'[t + j, c] (so w[c, K-1] multiplies
// the current token), out = C * conv, and the state becomes the last K-1 rows of x'
// (src/models/lfm3/lfm3_decoder.cpp:94-111; src/backend/cpu_ref/ops.cpp:447-471). Taps
// that reach before a sequence's first token of this step come from that sequence's
// state row, never from the neighbouring sequence's tokens. g is rounded to the
// activation type before use, as it is when it is kept in the state, so cutting a
// sequence into steps changes nothing.
//
// Taps are passed transposed, w_t[j, c], float32. The state is [slots, K-1, H].
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ float gated(const T* __restrict__ bcx, int64_t ld, int64_t t, int c, int H) {
    const T* row = bcx + t * ld;
    return to_f32(from_f32<T>(to_f32(row[c]) * to_f32(row[2 * H + c])));
}

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ bcx, int64_t ld, const float* __restrict__ w_t,
                                  const float* __restrict__ bias, const T* __restrict__ state,
                                  const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ cu_seqlens,
                                  const int32_t* __restrict__ slots, T* __restrict__ out, int Tn, int H, int K) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)Tn * H) return;
    const int t = (int)(idx / H), c = (int)(idx % H);
    const int seq = seq_of_token[t];
    const int first = cu_seqlens[seq];
    const int t_local = t - first;
    const T* st = state + (int64_t)slots[seq] * (K - 1) * H;
    float acc = bias != nullptr ? bias[c] : 0.0f;
    for (int j = 0; j < K; ++j) {
        const int r = t_local + j;   // row of x'
        const float v = r < K - 1 ? to_f32(st[(int64_t)r * H + c]) : gated(bcx, ld, (int64_t)first + r - (K - 1), c, H);
        acc = fmaf(w_t[(int64_t)j * H + c], v, acc);
    }
    out[idx] = from_f32<T>(to_f32(bcx[(int64_t)t * ld + H + c]) * acc);
}

// One thread per (sequence, channel) walks the K-1 state rows in ascending order: row a
// takes x'[a + T_i], which lies further on, so nothing is read after it was overwritten.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ bcx, int64_t ld, T* __restrict__ state,
                                        const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                                        int n_seqs, int H, int K) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)n_seqs * H) return;
    const int seq = (int)(idx / H), c = (int)(idx % H);
    const int first = cu_seqlens[seq];
    const int Ti = cu_seqlens[seq + 1] - first;
    T* st = state + (int64_t)slots[seq] * (K - 1) * H;
    for (int a = 0; a < K - 1; ++a) {
        const int r = a + Ti;
        const T v = r < K - 1 ? st[(int64_t)r * H + c]
                              : from_f32<T>(gated(bcx, ld, (int64_t)first + r - (K - 1), c, H));
        st[(int64_t)a * H + c] = v;
    }
}

}  // namespace

XS_API int xs_short_conv(const void* bcx, int64_t ld, const float* w_t, const float* bias, void* state,
                         const int32_t* seq_of_token, const int32_t* cu_seqlens, const int32_t* slots, void* out,
                         int T, int n_seqs, int H, int K, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(H > 0 && K >= 2 && n_seqs > 0 && ld >= 3 * (int64_t)H, "short_conv: width %d, %d taps, %d sequences", H, K, n_seqs);
    const int blocks = ceil_div_i((int64_t)T * H, 256);
    const int blocks2 = ceil_div_i((int64_t)n_seqs * H, 256);
    XS_DISPATCH_DTYPE(dtype, TT, {
        short_conv_kernel<TT><<<blocks, 256, 0, stream>>>((const TT*)bcx, ld, w_t, bias, (const TT*)state,
                                                          seq_of_token, cu_seqlens, slots, (TT*)out, T, H, K);
        short_conv_state_kernel<TT><<<blocks2, 256, 0, stream>>>((const TT*)bcx, ld, (TT*)state, cu_seqlens, slots,
                                                                 n_seqs, H, K);
    });
    XS_LAUNCH_CHECK("short_conv");
    return 0;
}
