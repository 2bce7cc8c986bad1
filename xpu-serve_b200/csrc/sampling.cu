// Next-token choice on the device: argmax, temperature / top-k / top-p / min-p sampling,
// repetition / presence / frequency penalties.
//
// Meaning of the parameters follows the reference's sampler (src/engine/sampler.cpp:20-132):
//   weight(t) = exp((logit[t] - max) / temperature)
//   candidates in descending logit order (ties: the lower token id first)
//   top_k > 0 keeps the first k; `total` is the weight of those
//   the list ends before the first weight < min_p, and after the first candidate at which
//   kept / total >= top_p (when top_p < 1)
//   a token is drawn from the kept candidates in proportion to their weights.
// The kept set is found without sorting, by radix selection over 64-bit keys (ordered
// logit bits, then inverted token id), and the draw walks the kept tokens in vocabulary
// order with the uniform u in [0, 1) that (seed, counter) gives (xs_uniform below), which
// is the same distribution as walking them in sorted order.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// u in [0, 1) with 53 random bits: two rounds of the splitmix64 finaliser over seed and counter.
__host__ __device__ __forceinline__ double uniform_from(uint64_t seed, uint64_t counter) {
    const uint64_t a = mix64(seed + 0x9E3779B97F4A7C15ull);
    const uint64_t b = mix64(a ^ (counter * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
    return (double)(b >> 11) * (1.0 / 9007199254740992.0);
}

__device__ __forceinline__ uint32_t ordered_bits(float v) {   // larger float -> larger unsigned
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ uint64_t key_of(float logit, int token) {
    return ((uint64_t)ordered_bits(logit) << 32) | (uint64_t)(0xFFFFFFFFu - (uint32_t)token);
}

__device__ __forceinline__ double block_sum_f64(double v, double* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = (threadIdx.x & 31) < (blockDim.x >> 5) ? scratch[threadIdx.x & 31] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

struct ArgBest {
    float v;
    int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// Largest value of a row and the lowest index that has it (NaN never wins). All threads get it.
__device__ ArgBest block_argmax(const float* __restrict__ row, int V, ArgBest* scratch) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int t = threadIdx.x; t < V; t += blockDim.x) best = better(best, ArgBest{row[t], t});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = best;
    __syncthreads();
    ArgBest r = (threadIdx.x & 31) < (blockDim.x >> 5) ? scratch[threadIdx.x & 31] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
        r = better(r, other);
    }
    if (r.i == 0x7fffffff) r.i = 0;   // a row of NaN or -inf
    return r;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int64_t ld, int V, int32_t* __restrict__ out) {
    __shared__ ArgBest scratch[32];
    const ArgBest r = block_argmax(logits + (int64_t)blockIdx.x * ld, V, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

// Wide rows, few of them: each row is cut into `parts` pieces so that more than a handful of SMs
// read it. packed[row] = max over pieces of (ordered value bits << 32 | ~index): the largest value
// wins, and among equals the lowest index. out[row] is decoded by argmax_finish_kernel.
__global__ void argmax_part_kernel(const float* __restrict__ logits, int64_t ld, int V, int parts,
                                   unsigned long long* __restrict__ packed) {
    __shared__ ArgBest scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, part = blockIdx.x;
    const int per = (V + parts - 1) / parts;
    const int begin = min(V, part * per), count = min(V, begin + per) - begin;
    if (count <= 0) return;
    ArgBest r = block_argmax(logits + (int64_t)row * ld + begin, count, scratch);
    if (threadIdx.x == 0) {
        const float v = r.v != r.v ? -INFINITY : r.v;
        const unsigned long long key = ((unsigned long long)ordered_bits(v) << 32) |
                                       (unsigned long long)(0xFFFFFFFFu - (unsigned)(begin + r.i));
        atomicMax(&packed[row], key);
    }
}
__global__ void argmax_finish_kernel(unsigned long long* __restrict__ packed, int n, int32_t* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = (int32_t)(0xFFFFFFFFu - (unsigned)(packed[i] & 0xFFFFFFFFull));
    packed[i] = 0ull;      // ready for the next call
}


// Radix descent, most significant byte first, over the keys >= `floor_key`.
// by_count: the key of rank `target_count` (1-based) in descending order.
// else:     the largest key K such that the weight of {keys >= K} reaches `target_mass`.
// If the target is never reached the smallest eligible key is returned.
__device__ uint64_t radix_select(const float* __restrict__ row, int V, float max_logit, float inv_temp,
                                 uint64_t floor_key, bool by_count, long long target_count, double target_mass,
                                 unsigned int* hist_count, double* hist_mass, uint64_t* shared_key,
                                 long long* shared_count, double* shared_mass) {
    uint64_t prefix = 0;
    long long above_count = 0;
    double above_mass = 0.0;
    for (int pass = 7; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            hist_count[b] = 0;
            hist_mass[b] = 0.0;
        }
        __syncthreads();
        const uint64_t hi_mask = pass == 7 ? 0ull : (~0ull << (shift + 8));
        for (int t = threadIdx.x; t < V; t += blockDim.x) {
            const float l = row[t];
            const uint64_t key = key_of(l, t);
            if (key < floor_key || (key & hi_mask) != prefix) continue;
            const int digit = (int)((key >> shift) & 0xFF);
            atomicAdd(&hist_count[digit], 1u);
            if (!by_count) atomicAdd(&hist_mass[digit], (double)expf((l - max_logit) * inv_temp));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            long long c = above_count;
            double m = above_mass;
            int chosen = -1;
            for (int b = 255; b >= 0; --b) {
                if (hist_count[b] == 0) continue;
                const long long c2 = c + hist_count[b];
                const double m2 = m + hist_mass[b];
                chosen = b;   // the lowest non-empty bucket so far: where an unreachable target lands
                if (by_count ? (c2 >= target_count) : (m2 >= target_mass)) break;
                c = c2;
                m = m2;
            }
            if (chosen < 0) chosen = 0;
            *shared_key = prefix | ((uint64_t)chosen << shift);
            *shared_count = c;
            *shared_mass = m;
        }
        __syncthreads();
        prefix = *shared_key;
        above_count = *shared_count;
        above_mass = *shared_mass;
        __syncthreads();
    }
    return prefix;
}

// One block per row.
__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t ld, int V, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const uint64_t* __restrict__ seeds, const uint64_t* __restrict__ counters, int32_t* __restrict__ out) {
    __shared__ ArgBest arg_scratch[32];
    __shared__ double sum_scratch[32];
    __shared__ unsigned int hist_count[256];
    __shared__ double hist_mass[256];
    __shared__ uint64_t shared_key;
    __shared__ long long shared_count;
    __shared__ double shared_mass;
    __shared__ double chunk_sum[kThreads];
    __shared__ int result;

    const int rowi = blockIdx.x;
    const float* row = logits + (int64_t)rowi * ld;
    const ArgBest top = block_argmax(row, V, arg_scratch);
    const float temp = temperature[rowi];
    const int k = top_k[rowi];
    if (!(temp > 0.0f) || k == 1) {   // greedy (src/engine/sampler.h:36)
        if (threadIdx.x == 0) out[rowi] = top.i;
        return;
    }
    const float inv_temp = 1.0f / temp;
    const float p_cut = top_p[rowi];
    const float w_cut = min_p[rowi];

    uint64_t floor_key = 0;   // keys below it are not candidates
    if (k > 0 && k < V) {
        floor_key = radix_select(row, V, top.v, inv_temp, 0, true, k, 0.0, hist_count, hist_mass, &shared_key,
                                 &shared_count, &shared_mass);
    }
    if (p_cut < 1.0f) {
        double mass = 0.0;   // `total`: the weight of the top-k candidates
        for (int t = threadIdx.x; t < V; t += blockDim.x) {
            const float l = row[t];
            if (key_of(l, t) >= floor_key) mass += (double)expf((l - top.v) * inv_temp);
        }
        mass = block_sum_f64(mass, sum_scratch);
        const uint64_t p_key = radix_select(row, V, top.v, inv_temp, floor_key, false, 0, (double)p_cut * mass,
                                            hist_count, hist_mass, &shared_key, &shared_count, &shared_mass);
        floor_key = p_key > floor_key ? p_key : floor_key;
    }

    // Kept: key >= floor_key and weight >= min_p (the likeliest token always stays).
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int begin = min(V, (int)threadIdx.x * per), end = min(V, begin + per);
    double mine = 0.0;
    for (int t = begin; t < end; ++t) {
        const float l = row[t];
        const float w = expf((l - top.v) * inv_temp);
        if (key_of(l, t) >= floor_key && (w >= w_cut || t == top.i)) mine += (double)w;
    }
    chunk_sum[threadIdx.x] = mine;
    if (threadIdx.x == 0) result = -1;
    __syncthreads();
    if (threadIdx.x == 0) {   // exclusive prefix over the chunks, in place
        double run = 0.0;
        for (int i = 0; i < (int)blockDim.x; ++i) {
            const double s = chunk_sum[i];
            chunk_sum[i] = run;
            run += s;
        }
        shared_mass = run;
    }
    __syncthreads();
    const double total = shared_mass;
    const double target = uniform_from(seeds[rowi], counters[rowi]) * total;
    const double before = chunk_sum[threadIdx.x];
    if (mine > 0.0 && target >= before && target < before + mine) {
        double left = target - before;
        int pick = -1, last = -1;
        for (int t = begin; t < end; ++t) {
            const float l = row[t];
            const float w = expf((l - top.v) * inv_temp);
            if (!(key_of(l, t) >= floor_key && (w >= w_cut || t == top.i))) continue;
            last = t;
            if (left < (double)w) {
                pick = t;
                break;
            }
            left -= (double)w;
        }
        result = pick >= 0 ? pick : last;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[rowi] = result >= 0 ? result : top.i;   // rounding put the target past the end
}

// logits[r, t] for seen tokens: divided (positive) or multiplied (negative) by the repetition
// penalty; for generated tokens: minus presence + frequency * count (sampler.cpp:20-47).
__global__ void penalties_kernel(float* __restrict__ logits, int64_t ld, int V, const uint8_t* __restrict__ seen,
                                 const int32_t* __restrict__ gen_count, const int32_t* __restrict__ state_rows,
                                 const float* __restrict__ repetition, const float* __restrict__ presence,
                                 const float* __restrict__ frequency) {
    const int r = blockIdx.y;
    const int64_t srow = state_rows[r];
    const float rp = repetition[r], pp = presence[r], fp = frequency[r];
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < V; t += gridDim.x * blockDim.x) {
        float l = logits[(int64_t)r * ld + t];
        if (rp != 1.0f && seen[srow * V + t]) l = l > 0.0f ? l / rp : l * rp;
        const int c = gen_count[srow * V + t];
        if (c > 0) l -= pp + fp * (float)c;
        logits[(int64_t)r * ld + t] = l;
    }
}

// seen[row, token] = 1; when `generated`, gen_count[row, token] += 1.
__global__ void note_tokens_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ rows_of_token,
                                   int n, int V, uint8_t* __restrict__ seen, int32_t* __restrict__ gen_count,
                                   int generated) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = tokens[i];
    if (t < 0 || t >= V) return;
    const int64_t at = (int64_t)rows_of_token[i] * V + t;
    seen[at] = 1;
    if (generated) atomicAdd(&gen_count[at], 1);
}

}  // namespace

XS_API double xs_uniform(uint64_t seed, uint64_t counter) { return uniform_from(seed, counter); }

// `packed`: n zeroed 64-bit words of scratch for wide rows (left zeroed again), or null.
XS_API int xs_argmax(const float* logits, int64_t ld, int n, int V, int32_t* out, unsigned long long* packed,
                     cudaStream_t stream) {
    if (n == 0) return 0;
    XS_REQUIRE(n > 0 && V > 0 && ld >= V, "argmax: %d rows of %d", n, V);
    if (V >= 16384 && n <= 65535 && packed != nullptr) {
        const int parts = min(32, V / 4096);
        xs_launch(argmax_part_kernel, dim3(parts, n), dim3(256), 0, stream, logits, ld, V, parts, packed);
        xs_launch(argmax_finish_kernel, dim3(ceil_div_i(n, 128)), dim3(128), 0, stream, packed, n, out);
        XS_LAUNCH_CHECK("argmax");
        return 0;
    }
    argmax_kernel<<<n, V >= 4096 ? 1024 : 256, 0, stream>>>(logits, ld, V, out);
    XS_LAUNCH_CHECK("argmax");
    return 0;
}

XS_API int xs_sample(const float* logits, int64_t ld, int n, int V, const float* temperature, const int32_t* top_k,
                     const float* top_p, const float* min_p, const uint64_t* seeds, const uint64_t* counters,
                     int32_t* out, cudaStream_t stream) {
    if (n == 0) return 0;
    XS_REQUIRE(n > 0 && V > 0 && ld >= V, "sample: %d rows of %d", n, V);
    sample_kernel<<<n, kThreads, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p, seeds, counters, out);
    XS_LAUNCH_CHECK("sample");
    return 0;
}

XS_API int xs_apply_penalties(float* logits, int64_t ld, int n, int V, const uint8_t* seen, const int32_t* gen_count,
                              const int32_t* state_rows, const float* repetition, const float* presence,
                              const float* frequency, cudaStream_t stream) {
    if (n == 0) return 0;
    XS_REQUIRE(n > 0 && V > 0 && ld >= V && n <= 65535, "penalties: %d rows of %d", n, V);
    const dim3 grid(min(ceil_div_i(V, 256), 64), n);
    penalties_kernel<<<grid, 256, 0, stream>>>(logits, ld, V, seen, gen_count, state_rows, repetition, presence,
                                               frequency);
    XS_LAUNCH_CHECK("penalties");
    return 0;
}

XS_API int xs_note_tokens(const int32_t* tokens, const int32_t* rows_of_token, int n, int V, uint8_t* seen,
                          int32_t* gen_count, int generated, cudaStream_t stream) {
    if (n == 0) return 0;
    note_tokens_kernel<<<ceil_div_i(n, 256), 256, 0, stream>>>(tokens, rows_of_token, n, V, seen, gen_count, generated);
    XS_LAUNCH_CHECK("note_tokens");
    return 0;
}
