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
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

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

// Calls f(logit, token) for the tokens [from, V) of the row, tokens dealt to the block's threads in turn, eight loads of a
// thread in flight at a time (a row is read from L2: one load at a time would be one latency per token).
template <typename F>
__device__ __forceinline__ void for_row_strided(const float* __restrict__ row, int from, int V, F&& f) {
    const int step = (int)blockDim.x;
    for (int t0 = from + threadIdx.x; t0 < V; t0 += step * 8) {
        float l[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int t = t0 + u * step;
            l[u] = t < V ? __ldg(row + t) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int t = t0 + u * step;
            if (t < V) f(l[u], t);
        }
    }
}

// The same for the tokens [begin, end) that one thread owns, in token order; 16-byte loads when `vec`.
template <typename F>
__device__ __forceinline__ void for_chunk(const float* __restrict__ row, int begin, int end, bool vec, F&& f) {
    if (vec) {
        for (int t0 = begin; t0 < end; t0 += 16) {
            float4 l[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                l[u] = t0 + 4 * u < end ? __ldg(reinterpret_cast<const float4*>(row + t0 + 4 * u)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int t = t0 + 4 * u;
                if (t < end) {
                    if (!f(l[u].x, t) || !f(l[u].y, t + 1) || !f(l[u].z, t + 2) || !f(l[u].w, t + 3)) return;
                }
            }
        }
        return;
    }
    for (int t = begin; t < end; ++t)
        if (!f(__ldg(row + t), t)) return;
}

struct ArgBest {
    float v;
    int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// Largest value of a row and the lowest index that has it (NaN never wins). All threads get it.
__device__ ArgBest block_argmax(const float* __restrict__ row, int from, int V, ArgBest* scratch) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for_row_strided(row, from, V, [&](float l, int t) { best = better(best, ArgBest{l, t}); });
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
    if (r.i == 0x7fffffff) r.i = from;   // a row of NaN or -inf
    return r;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int64_t ld, int V, int32_t* __restrict__ out) {
    __shared__ ArgBest scratch[32];
    const ArgBest r = block_argmax(logits + (int64_t)blockIdx.x * ld, 0, V, scratch);
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
    ArgBest r = block_argmax(logits + (int64_t)row * ld + begin, 0, count, scratch);
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


// Weights are added up as 64-bit fixed point (2^-40 of the largest weight, which is 1): integer sums do not
// depend on the order in which threads add, so a row's kept set and draw are the same in every run.
constexpr int kSub = 32;                          // histograms a block keeps, one per warp
constexpr double kFixOne = 1099511627776.0;       // 2^40
constexpr int kMaxVocab = 1 << 22;                // 2^22 weights of at most 2^40 stay below 2^63

__device__ __forceinline__ unsigned long long fix_of(float w) { return __double2ull_rz((double)w * kFixOne); }

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long t = (threadIdx.x & 31) < (blockDim.x >> 5) ? scratch[threadIdx.x & 31] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// Exclusive prefix of v over the block's threads in thread order; *total gets the sum. scratch: 33 words.
__device__ __forceinline__ unsigned long long block_exclusive_scan_u64(unsigned long long v, unsigned long long* scratch,
                                                                       unsigned long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        const unsigned long long w = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0ull;
        unsigned long long winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += up;
        }
        scratch[lane] = winc - w;                 // what the warps before this one hold
        if (lane == 31) scratch[32] = winc;
    }
    __syncthreads();
    *total = scratch[32];
    return scratch[warp] + inc - v;
}

// A row is shared by the CTAs of a thread-block cluster: each reads its part of the vocabulary, and what the
// parts have to know of one another (the largest logit, a pass's 256 bucket sums, the sums of the kept weights)
// they read from one another's shared memory. With 8 or 64 rows and one CTA a row most of the device would idle
// while each CTA reads its 65,536 logits a dozen times over.
struct RowShare {
    unsigned int count[256];            // this CTA's part of a pass's histogram
    unsigned long long mass[256];
    ArgBest best;
    unsigned long long sum;
    uint64_t key;
    int key_set;
};

struct RadixScratch {
    unsigned int* sub_count;            // [kSub][256]
    unsigned int* sub_mass_lo;          // [kSub][256]: a warp's mass in a bucket is hi * 2^32 + lo
    unsigned int* sub_mass_hi;          // [kSub][256]
    RowShare* share;                    // this CTA's
    unsigned int* all_count;            // [256]: the whole row's
    unsigned long long* all_mass;       // [256]
    uint64_t* key;
    long long* above_count;
    unsigned long long* above_mass;
    unsigned int* left;                 // keys in the bucket the walk chose
};

__device__ __forceinline__ const RowShare* share_of(cg::cluster_group& cluster, RowShare* mine, unsigned int rank) {
    return cluster.map_shared_rank(mine, rank);
}

// Sum of every CTA's v, in rank order, the same in all of them.
__device__ __forceinline__ unsigned long long cluster_sum_u64(cg::cluster_group& cluster, RowShare* share,
                                                              unsigned long long v, unsigned long long* before) {
    if (threadIdx.x == 0) share->sum = v;
    cluster.sync();
    unsigned long long total = 0, lower = 0;
    for (unsigned int r = 0; r < cluster.num_blocks(); ++r) {
        const unsigned long long x = share_of(cluster, share, r)->sum;
        if (r < cluster.block_rank()) lower += x;
        total += x;
    }
    cluster.sync();                     // everybody has read before anybody writes the next
    if (before != nullptr) *before = lower;
    return total;
}

// Radix descent, most significant byte first, over the keys >= `floor_key` of the whole row; this CTA reads the
// tokens [lo, hi) of it. Every CTA of the cluster returns the same key.
// by_count: the key of rank `target_count` (1-based) in descending order.
// else:     the largest key K such that the weight of {keys >= K} reaches `target_mass` (in fixed point).
// If the target is never reached the smallest eligible key is returned.
// Every warp counts into a histogram of its own (all 65,536 logits of a row share a handful of leading bytes: one
// histogram for the block would serialise a thousand threads on a few words), a thread per bucket adds the warps'
// histograms, and one warp of every CTA adds the CTAs' and walks the 256 buckets, eight a lane.
__device__ uint64_t radix_select(cg::cluster_group& cluster, const float* __restrict__ row, int lo, int hi_tok,
                                 float max_logit, float inv_temp, uint64_t floor_key, bool by_count,
                                 long long target_count, double target_mass, const RadixScratch& sc) {
    uint64_t prefix = 0;
    long long above_count = 0;
    unsigned long long above_mass = 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned int ranks = cluster.num_blocks();
    unsigned int* my_count = sc.sub_count + (warp % kSub) * 256;
    unsigned int* my_lo = sc.sub_mass_lo + (warp % kSub) * 256;
    unsigned int* my_hi = sc.sub_mass_hi + (warp % kSub) * 256;
    for (int pass = 7; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int b = threadIdx.x; b < kSub * 256; b += blockDim.x) {
            sc.sub_count[b] = 0;
            if (!by_count) {
                sc.sub_mass_lo[b] = 0;
                sc.sub_mass_hi[b] = 0;
            }
        }
        __syncthreads();
        const uint64_t hi_mask = pass == 7 ? 0ull : (~0ull << (shift + 8));
        for_row_strided(row, lo, hi_tok, [&](float l, int t) {
            const uint64_t key = key_of(l, t);
            if (key < floor_key || (key & hi_mask) != prefix) return;
            const int digit = (int)((key >> shift) & 0xFF);
            atomicAdd(&my_count[digit], 1u);
            if (!by_count) {
                // a 64-bit sum out of 32-bit adds (the kind shared memory does by itself): the low word, one more
                // in the high word whenever the low word wraps, and the weight's own high word (zero below 2^-8)
                const unsigned long long f = fix_of(expf((l - max_logit) * inv_temp));
                const unsigned int flo = (unsigned int)f, fhi = (unsigned int)(f >> 32);
                const unsigned int old = atomicAdd(&my_lo[digit], flo);
                const unsigned int carry = old + flo < old ? 1u : 0u;
                if (fhi + carry != 0u) atomicAdd(&my_hi[digit], fhi + carry);
            }
        });
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned int c = 0;
            unsigned long long m = 0;
#pragma unroll 8
            for (int w = 0; w < kSub; ++w) {
                c += sc.sub_count[w * 256 + b];
                if (!by_count)
                    m += ((unsigned long long)sc.sub_mass_hi[w * 256 + b] << 32) + sc.sub_mass_lo[w * 256 + b];
            }
            sc.share->count[b] = c;
            sc.share->mass[b] = m;
        }
        cluster.sync();
        // a thread per bucket adds the CTAs' sums (its loads from the other CTAs' shared memory all in flight at once)
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned int c = 0;
            unsigned long long m = 0;
            for (unsigned int r = 0; r < ranks; ++r) {
                const RowShare* other = share_of(cluster, sc.share, r);
                c += other->count[b];
                if (!by_count) m += other->mass[b];
            }
            sc.all_count[b] = c;
            sc.all_mass[b] = m;
        }
        __syncthreads();
        if (warp == 0) {
            // lane L owns buckets 255 - 8 L down to 248 - 8 L: lane 0 the largest digits
            const int hi = 255 - 8 * lane;
            long long bc[8];
            unsigned long long bm[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bc[j] = sc.all_count[hi - j];
                bm[j] = sc.all_mass[hi - j];
            }
            long long c = 0;
            unsigned long long m = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                c += bc[j];
                m += bm[j];
            }
            long long c_inc = c;
            unsigned long long m_inc = m;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long cu = __shfl_up_sync(0xffffffffu, c_inc, o);
                const unsigned long long mu = __shfl_up_sync(0xffffffffu, m_inc, o);
                if (lane >= o) {
                    c_inc += cu;
                    m_inc += mu;
                }
            }
            c = above_count + c_inc - c;          // what lies above this lane's buckets
            m = above_mass + m_inc - m;
            int found = -1, low = -1;
            long long found_n = 0, low_n = 0;
            long long found_c = 0, low_c = 0;
            unsigned long long found_m = 0, low_m = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const long long n = bc[j];
                if (n == 0 || found >= 0) continue;
                low = hi - j;                      // the lowest non-empty bucket so far, and what lies above it
                low_n = n;
                low_c = c;
                low_m = m;
                const long long c2 = c + n;
                const unsigned long long m2 = m + bm[j];
                if (by_count ? (c2 >= target_count) : ((double)m2 >= target_mass)) {
                    found = hi - j;
                    found_n = n;
                    found_c = c;
                    found_m = m;
                }
                c = c2;
                m = m2;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, found >= 0);
            const unsigned any = __ballot_sync(0xffffffffu, low >= 0);
            if (hit != 0u) {
                if (lane == __ffs(hit) - 1) {
                    *sc.key = prefix | ((uint64_t)found << shift);
                    *sc.above_count = found_c;
                    *sc.above_mass = found_m;
                    *sc.left = found_n == 1 ? 1u : 2u;
                }
            } else if (any != 0u) {               // an unreachable target lands on the lowest non-empty bucket
                if (lane == 31 - __clz(any)) {
                    *sc.key = prefix | ((uint64_t)low << shift);
                    *sc.above_count = low_c;
                    *sc.above_mass = low_m;
                    *sc.left = low_n == 1 ? 1u : 2u;
                }
            } else if (lane == 0) {
                *sc.key = prefix;
                *sc.above_count = above_count;
                *sc.above_mass = above_mass;
                *sc.left = 0;
            }
            if (lane == 0) sc.share->key_set = 0;
        }
        cluster.sync();                           // the histograms have been read: the next pass may clear them
        prefix = *sc.key;
        above_count = *sc.above_count;
        above_mass = *sc.above_mass;
        const unsigned int left = *sc.left;
        if (left == 1 && pass > 0) {
            // one key has this prefix: it is the answer, and whoever holds it says so (the remaining passes would
            // each read the whole row to learn one more byte of it)
            const uint64_t got_mask = ~0ull << shift;
            for_row_strided(row, lo, hi_tok, [&](float l, int t) {
                const uint64_t key = key_of(l, t);
                if (key >= floor_key && (key & got_mask) == prefix) {
                    sc.share->key = key;
                    sc.share->key_set = 1;
                }
            });
            cluster.sync();
            for (unsigned int r = 0; r < ranks; ++r) {
                const RowShare* other = share_of(cluster, sc.share, r);
                if (other->key_set) prefix = other->key;
            }
            cluster.sync();
            return prefix;
        }
        __syncthreads();
    }
    return prefix;
}

constexpr size_t kSampleSmem = (size_t)kSub * 256 * 3 * sizeof(unsigned int);

// One cluster of CTAs per row (gridDim.x = rows x cluster size).
__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t ld, int V, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const uint64_t* __restrict__ seeds, uint64_t* __restrict__ counters, int advance, int32_t* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    __shared__ ArgBest arg_scratch[32];
    __shared__ unsigned long long sum_scratch[33];
    __shared__ RowShare share;
    __shared__ unsigned int all_count[256];
    __shared__ unsigned long long all_mass[256];
    __shared__ uint64_t shared_key;
    __shared__ long long shared_count;
    __shared__ unsigned long long shared_mass;
    __shared__ unsigned int shared_left;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned int ranks = cluster.num_blocks(), rank = cluster.block_rank();
    RadixScratch sc;
    sc.sub_count = reinterpret_cast<unsigned int*>(sample_smem);
    sc.sub_mass_lo = sc.sub_count + kSub * 256;
    sc.sub_mass_hi = sc.sub_mass_lo + kSub * 256;
    sc.share = &share;
    sc.all_count = all_count;
    sc.all_mass = all_mass;
    sc.key = &shared_key;
    sc.above_count = &shared_count;
    sc.above_mass = &shared_mass;
    sc.left = &shared_left;

    const int rowi = blockIdx.x / ranks;
    const float* row = logits + (int64_t)rowi * ld;
    const uint64_t draw = counters[rowi];       // every CTA of the row reads it before the first cluster-wide barrier
    // this CTA's part of the vocabulary, a multiple of 4 tokens long (16-byte loads below)
    const int part = ((V + (int)ranks - 1) / (int)ranks + 3) & ~3;
    const int lo = min(V, (int)rank * part), hi = min(V, lo + part);

    const ArgBest mine_best = block_argmax(row, lo, hi, arg_scratch);
    if (threadIdx.x == 0) share.best = lo < hi ? mine_best : ArgBest{-INFINITY, 0x7fffffff};
    cluster.sync();
    ArgBest top{-INFINITY, 0x7fffffff};
    for (unsigned int r = 0; r < ranks; ++r) top = better(top, share_of(cluster, &share, r)->best);
    if (top.i == 0x7fffffff) top.i = 0;   // a row of NaN or -inf
    cluster.sync();
    // the row's draw counter moves on here, on the device (greedy rows too: a counter counts steps), once all have read it
    if (advance && threadIdx.x == 0 && rank == 0) counters[rowi] = draw + 1;
    const float temp = temperature[rowi];
    const int k = top_k[rowi];
    if (!(temp > 0.0f) || k == 1) {   // greedy (src/engine/sampler.h:36)
        if (threadIdx.x == 0 && rank == 0) out[rowi] = top.i;
        return;
    }
    const float inv_temp = 1.0f / temp;
    const float p_cut = top_p[rowi];
    const float w_cut = min_p[rowi];

    uint64_t floor_key = 0;   // keys below it are not candidates
    if (k > 0 && k < V) floor_key = radix_select(cluster, row, lo, hi, top.v, inv_temp, 0, true, k, 0.0, sc);
    if (p_cut < 1.0f) {
        unsigned long long mass = 0;   // `total`: the weight of the top-k candidates
        for_row_strided(row, lo, hi, [&](float l, int t) {
            if (key_of(l, t) >= floor_key) mass += fix_of(expf((l - top.v) * inv_temp));
        });
        mass = block_sum_u64(mass, sum_scratch);
        mass = cluster_sum_u64(cluster, &share, mass, nullptr);
        const uint64_t p_key = radix_select(cluster, row, lo, hi, top.v, inv_temp, floor_key, false, 0,
                                            (double)p_cut * (double)mass, sc);
        floor_key = p_key > floor_key ? p_key : floor_key;
    }

    // Kept: key >= floor_key and weight >= min_p (the likeliest token always stays). The draw walks the kept
    // tokens in vocabulary order: CTA after CTA, thread after thread, each thread a run of neighbouring tokens.
    const int per = ((hi - lo + (int)blockDim.x - 1) / (int)blockDim.x + 3) & ~3;
    const int begin = min(hi, lo + (int)threadIdx.x * per), end = min(hi, begin + per);
    const bool vec = V % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    unsigned long long mine = 0;
    for_chunk(row, begin, end, vec, [&](float l, int t) {
        const float w = expf((l - top.v) * inv_temp);
        if (key_of(l, t) >= floor_key && (w >= w_cut || t == top.i)) mine += fix_of(w);
        return true;
    });
    if (threadIdx.x == 0 && rank == 0) out[rowi] = top.i;     // stands only if every kept weight rounded to zero
    unsigned long long cta_total = 0, lower = 0;
    const unsigned long long before_in_cta = block_exclusive_scan_u64(mine, sum_scratch, &cta_total);
    const unsigned long long total = cluster_sum_u64(cluster, &share, cta_total, &lower);   // also orders the write above
    const unsigned long long before = lower + before_in_cta;
    unsigned long long target = __double2ull_rz(uniform_from(seeds[rowi], draw) * (double)total);
    if (total > 0 && target >= total) target = total - 1;
    if (mine > 0 && target >= before && target < before + mine) {
        unsigned long long left = target - before;
        int pick = -1, last = -1;
        for_chunk(row, begin, end, vec, [&](float l, int t) {
            const float w = expf((l - top.v) * inv_temp);
            if (!(key_of(l, t) >= floor_key && (w >= w_cut || t == top.i))) return true;
            last = t;
            const unsigned long long f = fix_of(w);
            if (left < f) {
                pick = t;
                return false;
            }
            left -= f;
            return true;
        });
        out[rowi] = pick >= 0 ? pick : last;
    }
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
                     const float* top_p, const float* min_p, const uint64_t* seeds, uint64_t* counters, int advance,
                     int32_t* out, cudaStream_t stream) {
    if (n == 0) return 0;
    XS_REQUIRE(n > 0 && V > 0 && V <= kMaxVocab && ld >= V, "sample: %d rows of %d (at most %d)", n, V, kMaxVocab);
    static bool opted = false;
    static int sms = 0;
    if (!opted) {
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSampleSmem);
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        opted = true;
    }
    // CTAs a row: 8, or fewer (4, 2) so that all rows' CTAs run at one time (a CTA of 1,024 threads has an SM to
    // itself; measured on B200 at 64 rows of 65,536 with top-p: 2 a row 96 us, 4 a row 108 us, 1 a row 111 us); one
    // when the rows alone fill the device or the vocabulary is small
    int ranks = 1;
    if (V >= 8192)
        for (ranks = 8; ranks > 1 && (int64_t)n * ranks > (int64_t)sms; ranks >>= 1) {}
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n * ranks));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSampleSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, V, temperature, top_k, top_p, min_p, seeds,
                                             counters, advance, out);
    XS_REQUIRE(e == cudaSuccess, "sample: launch failed: %s", cudaGetErrorString(e));
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
