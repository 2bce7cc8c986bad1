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
    pdl_launch_dependents();
    pdl_wait();
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
    pdl_launch_dependents();
    pdl_wait();
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

// ---- bfloat16, 8 channels a thread (16-byte loads and stores); H a multiple of 8.
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 v = __bfloat1622float2(p[k]);
        f[2 * k] = v.x;
        f[2 * k + 1] = v.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 raw;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    return raw;
}
// g = B * X of one token for 8 channels, rounded to bfloat16 as the state keeps it
__device__ __forceinline__ void gated8(const __nv_bfloat16* __restrict__ row, int c8, int H, float (&g)[8]) {
    float b[8], x[8];
    unpack8(*reinterpret_cast<const uint4*>(row + c8), b);
    unpack8(*reinterpret_cast<const uint4*>(row + 2 * H + c8), x);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = __bfloat162float(__float2bfloat16_rn(b[k] * x[k]));
}

__global__ void short_conv_bf16x8_kernel(const __nv_bfloat16* __restrict__ bcx, int64_t ld, const float* __restrict__ w_t,
                                         const float* __restrict__ bias, const __nv_bfloat16* __restrict__ state,
                                         const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ cu_seqlens,
                                         const int32_t* __restrict__ slots, __nv_bfloat16* __restrict__ out, int Tn, int H,
                                         int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int H8 = H >> 3;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)Tn * H8) return;
    const int t = (int)(idx / H8), c8 = (int)(idx % H8) * 8;
    const int seq = seq_of_token[t];
    const int first = cu_seqlens[seq];
    const int t_local = t - first;
    const __nv_bfloat16* st = state + (int64_t)slots[seq] * (K - 1) * H;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = bias != nullptr ? bias[c8 + k] : 0.0f;
    for (int j = 0; j < K; ++j) {
        const int r = t_local + j;
        float v[8];
        if (r < K - 1) unpack8(*reinterpret_cast<const uint4*>(st + (int64_t)r * H + c8), v);
        else gated8(bcx + ((int64_t)first + r - (K - 1)) * ld, c8, H, v);
        const float4 w0 = *reinterpret_cast<const float4*>(w_t + (int64_t)j * H + c8);
        const float4 w1 = *reinterpret_cast<const float4*>(w_t + (int64_t)j * H + c8 + 4);
        acc[0] = fmaf(w0.x, v[0], acc[0]); acc[1] = fmaf(w0.y, v[1], acc[1]);
        acc[2] = fmaf(w0.z, v[2], acc[2]); acc[3] = fmaf(w0.w, v[3], acc[3]);
        acc[4] = fmaf(w1.x, v[4], acc[4]); acc[5] = fmaf(w1.y, v[5], acc[5]);
        acc[6] = fmaf(w1.z, v[6], acc[6]); acc[7] = fmaf(w1.w, v[7], acc[7]);
    }
    float c[8];
    unpack8(*reinterpret_cast<const uint4*>(bcx + (int64_t)t * ld + H + c8), c);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= c[k];
    *reinterpret_cast<uint4*>(out + (int64_t)t * H + c8) = pack8(acc);
}

// Long prompts: a thread walks RUN neighbouring tokens of its 8 channels with the last KT-1 gated inputs in
// registers, so that B, C and X of a token are read once (not once per tap) and the taps once per thread.
// A run that lies inside one sequence (nearly all of them) asks for nothing by index but its first token's sequence:
// its loads do not wait for one another, four tokens' worth are in flight at a time. A run that crosses from one
// sequence into the next, or ends the step, goes token by token: at its first token, and wherever a sequence starts,
// the history is fetched as the plain kernel does (state rows, or earlier tokens of the same sequence). Both add up
// a token's taps in the plain kernel's order.
template <int KT, int RUN>
__global__ void __launch_bounds__(128) short_conv_bf16x8_run_kernel(
    const __nv_bfloat16* __restrict__ bcx, int64_t ld, const float* __restrict__ w_t, const float* __restrict__ bias,
    const __nv_bfloat16* __restrict__ state, const int32_t* __restrict__ seq_of_token,
    const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots, __nv_bfloat16* __restrict__ out, int Tn,
    int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int H8 = H >> 3;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int run = (int)(idx / H8), c8 = (int)(idx % H8) * 8;
    const int t0 = run * RUN;
    if (t0 >= Tn) return;
    const int t_last = min(t0 + RUN, Tn) - 1;
    const int seq0 = seq_of_token[t0], seq1 = seq_of_token[t_last];
    float w[KT][8], b0[8];
#pragma unroll
    for (int j = 0; j < KT; ++j) {
        const float4 w0 = *reinterpret_cast<const float4*>(w_t + (int64_t)j * H + c8);
        const float4 w1 = *reinterpret_cast<const float4*>(w_t + (int64_t)j * H + c8 + 4);
        w[j][0] = w0.x; w[j][1] = w0.y; w[j][2] = w0.z; w[j][3] = w0.w;
        w[j][4] = w1.x; w[j][5] = w1.y; w[j][6] = w1.z; w[j][7] = w1.w;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) b0[k] = bias != nullptr ? bias[c8 + k] : 0.0f;
    float hist[KT - 1][8];
    auto one_token = [&](const float (&g)[8], const float (&c)[8], int t) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float a = b0[k];
#pragma unroll
            for (int j = 0; j < KT - 1; ++j) a = fmaf(w[j][k], hist[j][k], a);   // taps in the plain kernel's order
            acc[k] = fmaf(w[KT - 1][k], g[k], a) * c[k];
        }
        *reinterpret_cast<uint4*>(out + (int64_t)t * H + c8) = pack8(acc);
#pragma unroll
        for (int j = 0; j + 1 < KT - 1; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) hist[j][k] = hist[j + 1][k];
#pragma unroll
        for (int k = 0; k < 8; ++k) hist[KT - 2][k] = g[k];
    };
    if (seq0 == seq1 && t_last == t0 + RUN - 1) {
        const int t_local = t0 - cu_seqlens[seq0];
        if (t_local >= KT - 1) {            // (the same for all threads of a run)
#pragma unroll
            for (int j = 0; j < KT - 1; ++j) gated8(bcx + (int64_t)(t0 + j - (KT - 1)) * ld, c8, H, hist[j]);
        } else {
            const __nv_bfloat16* st = state + (int64_t)slots[seq0] * (KT - 1) * H;
#pragma unroll
            for (int j = 0; j < KT - 1; ++j) {
                const int r = t_local + j;
                if (r < KT - 1) unpack8(*reinterpret_cast<const uint4*>(st + (int64_t)r * H + c8), hist[j]);
                else gated8(bcx + (int64_t)(t0 + j - (KT - 1)) * ld, c8, H, hist[j]);
            }
        }
#pragma unroll
        for (int i0 = 0; i0 < RUN; i0 += 4) {
            uint4 rb[4], rx[4], rc[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat16* row = bcx + (int64_t)(t0 + i0 + i) * ld + c8;
                rb[i] = *reinterpret_cast<const uint4*>(row);
                rc[i] = *reinterpret_cast<const uint4*>(row + H);
                rx[i] = *reinterpret_cast<const uint4*>(row + 2 * H);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float b[8], x[8], g[8], c[8];
                unpack8(rb[i], b);
                unpack8(rx[i], x);
                unpack8(rc[i], c);
#pragma unroll
                for (int k = 0; k < 8; ++k) g[k] = __bfloat162float(__float2bfloat16_rn(b[k] * x[k]));
                one_token(g, c, t0 + i0 + i);
            }
        }
        return;
    }
#pragma unroll 1
    for (int t = t0; t <= t_last; ++t) {
        const int seq = seq_of_token[t];
        const int first = cu_seqlens[seq];
        const int t_local = t - first;
        if (t == t0 || t_local == 0) {
            const __nv_bfloat16* st = state + (int64_t)slots[seq] * (KT - 1) * H;
#pragma unroll
            for (int j = 0; j < KT - 1; ++j) {
                const int r = t_local + j;
                if (r < KT - 1) unpack8(*reinterpret_cast<const uint4*>(st + (int64_t)r * H + c8), hist[j]);
                else gated8(bcx + ((int64_t)first + r - (KT - 1)) * ld, c8, H, hist[j]);
            }
        }
        float g[8], c[8];
        gated8(bcx + (int64_t)t * ld, c8, H, g);
        unpack8(*reinterpret_cast<const uint4*>(bcx + (int64_t)t * ld + H + c8), c);
        one_token(g, c, t);
    }
}

// Every sequence brings one token: the thread that owns (sequence, 8 channels) reads the state's
// K-1 rows, computes the output and writes the shifted state, in one kernel. The taps and the slot numbers are
// written by no kernel of a step (weights; the step's description, copied before the step's first kernel), so
// they are read before waiting for the kernel before this one, and the state's address is ready when the wait
// ends. The state itself is read after the wait: the kernel that wrote it last is this layer's own in the step
// before, and nothing but the chain of waits says that it is done.
template <int KT>
__global__ void short_conv_decode_bf16x8_kernel(const __nv_bfloat16* __restrict__ bcx, int64_t ld,
                                                const float* __restrict__ w_t, const float* __restrict__ bias,
                                                __nv_bfloat16* __restrict__ state, const int32_t* __restrict__ slots,
                                                __nv_bfloat16* __restrict__ out, int n_seqs, int H) {
    pdl_launch_dependents();
    const int H8 = H >> 3;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = idx < (int64_t)n_seqs * H8;
    const int seq = live ? (int)(idx / H8) : 0, c8 = live ? (int)(idx % H8) * 8 : 0;
    __nv_bfloat16* st = state + (int64_t)slots[seq] * (KT - 1) * H;
    float4 w0[KT], w1[KT];
#pragma unroll
    for (int j = 0; j < KT; ++j) {
        w0[j] = *reinterpret_cast<const float4*>(w_t + (int64_t)j * H + c8);
        w1[j] = *reinterpret_cast<const float4*>(w_t + (int64_t)j * H + c8 + 4);
    }
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = bias != nullptr ? bias[c8 + k] : 0.0f;
    pdl_wait();
    if (!live) return;
    uint4 old[KT - 1];
#pragma unroll
    for (int j = 0; j < KT - 1; ++j) old[j] = *reinterpret_cast<const uint4*>(st + (int64_t)j * H + c8);
    float g[8];
    gated8(bcx + (int64_t)seq * ld, c8, H, g);
#pragma unroll
    for (int j = 0; j < KT; ++j) {
        float v[8];
        if (j < KT - 1) {
            unpack8(old[j], v);
            if (j > 0) *reinterpret_cast<uint4*>(st + (int64_t)(j - 1) * H + c8) = old[j];   // row j moves to j - 1
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = g[k];
        }
        acc[0] = fmaf(w0[j].x, v[0], acc[0]); acc[1] = fmaf(w0[j].y, v[1], acc[1]);
        acc[2] = fmaf(w0[j].z, v[2], acc[2]); acc[3] = fmaf(w0[j].w, v[3], acc[3]);
        acc[4] = fmaf(w1[j].x, v[4], acc[4]); acc[5] = fmaf(w1[j].y, v[5], acc[5]);
        acc[6] = fmaf(w1[j].z, v[6], acc[6]); acc[7] = fmaf(w1[j].w, v[7], acc[7]);
    }
    *reinterpret_cast<uint4*>(st + (int64_t)(KT - 2) * H + c8) = pack8(g);
    float c[8];
    unpack8(*reinterpret_cast<const uint4*>(bcx + (int64_t)seq * ld + H + c8), c);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= c[k];
    *reinterpret_cast<uint4*>(out + (int64_t)seq * H + c8) = pack8(acc);
}

}  // namespace

// `all_single` != 0 promises that every sequence brings exactly one token (T == n_seqs).
XS_API int xs_short_conv(const void* bcx, int64_t ld, const float* w_t, const float* bias, void* state,
                         const int32_t* seq_of_token, const int32_t* cu_seqlens, const int32_t* slots, void* out,
                         int T, int n_seqs, int H, int K, int dtype, int all_single, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(H > 0 && K >= 2 && n_seqs > 0 && ld >= 3 * (int64_t)H, "short_conv: width %d, %d taps, %d sequences", H, K, n_seqs);
    XS_REQUIRE(!all_single || T == n_seqs, "short_conv: %d tokens for %d sequences of one token each", T, n_seqs);
    const bool vec = dtype == XS_BF16 && H % 8 == 0 && ld % 8 == 0 && (uintptr_t)bcx % 16 == 0 &&
                     (uintptr_t)state % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)w_t % 16 == 0;
    if (vec && all_single && K >= 2 && K <= 8) {
        const dim3 grid(ceil_div_i((int64_t)n_seqs * (H / 8), 128));
#define XS_CONV_DECODE(KT)                                                                                           \
    xs_launch(short_conv_decode_bf16x8_kernel<KT>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)bcx, ld, w_t, bias, \
              (__nv_bfloat16*)state, slots, (__nv_bfloat16*)out, n_seqs, H)
        switch (K) {
            case 2: XS_CONV_DECODE(2); break;
            case 3: XS_CONV_DECODE(3); break;
            case 4: XS_CONV_DECODE(4); break;
            case 5: XS_CONV_DECODE(5); break;
            case 6: XS_CONV_DECODE(6); break;
            case 7: XS_CONV_DECODE(7); break;       // the reference's default number of taps
            default: XS_CONV_DECODE(8); break;
        }
#undef XS_CONV_DECODE
        XS_LAUNCH_CHECK("short_conv_decode");
        return 0;
    }
    if (vec) {
        // runs of 8 tokens when that still makes 64 k threads (2,048 tokens of 2,048 channels), else runs of 4, else
        // (short steps) one thread a token
        const int64_t threads8 = (int64_t)ceil_div_i(T, 8) * (H / 8), threads4 = (int64_t)ceil_div_i(T, 4) * (H / 8);
        if (K >= 2 && K <= 8 && threads4 >= 64 * 1024) {
            const bool long_runs = threads8 >= 64 * 1024;
            const dim3 grid(ceil_div_i(long_runs ? threads8 : threads4, 128));
#define XS_CONV_RUN(KT)                                                                                              \
    do {                                                                                                             \
        if (long_runs)                                                                                               \
            short_conv_bf16x8_run_kernel<KT, 8><<<grid, 128, 0, stream>>>(                                            \
                (const __nv_bfloat16*)bcx, ld, w_t, bias, (const __nv_bfloat16*)state, seq_of_token, cu_seqlens, slots, \
                (__nv_bfloat16*)out, T, H);                                                                          \
        else                                                                                                         \
            short_conv_bf16x8_run_kernel<KT, 4><<<grid, 128, 0, stream>>>(                                            \
                (const __nv_bfloat16*)bcx, ld, w_t, bias, (const __nv_bfloat16*)state, seq_of_token, cu_seqlens, slots, \
                (__nv_bfloat16*)out, T, H);                                                                          \
    } while (0)
            switch (K) {
                case 2: XS_CONV_RUN(2); break;
                case 3: XS_CONV_RUN(3); break;
                case 4: XS_CONV_RUN(4); break;
                case 5: XS_CONV_RUN(5); break;
                case 6: XS_CONV_RUN(6); break;
                case 7: XS_CONV_RUN(7); break;       // the reference's default number of taps
                default: XS_CONV_RUN(8); break;
            }
#undef XS_CONV_RUN
        } else {
            short_conv_bf16x8_kernel<<<ceil_div_i((int64_t)T * (H / 8), 256), 256, 0, stream>>>(
                (const __nv_bfloat16*)bcx, ld, w_t, bias, (const __nv_bfloat16*)state, seq_of_token, cu_seqlens, slots,
                (__nv_bfloat16*)out, T, H, K);
        }
        short_conv_state_kernel<__nv_bfloat16><<<ceil_div_i((int64_t)n_seqs * H, 256), 256, 0, stream>>>(
            (const __nv_bfloat16*)bcx, ld, (__nv_bfloat16*)state, cu_seqlens, slots, n_seqs, H, K);
        XS_LAUNCH_CHECK("short_conv");
        return 0;
    }
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
