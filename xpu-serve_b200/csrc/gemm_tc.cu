// out[T, N] = x[T, K] . w[N, K]^T on Blackwell's fifth-generation tensor cores (tcgen05), bfloat16
// in, float32 accumulation in tensor memory.
//
// Orientation: the weight's rows ride the MMA's M side (128 rows a tile) and the tokens its N side
// (16 to 256 a tile), so the same kernel serves a prefill of thousands of tokens and a decode
// step of one token a sequence, where the product is a stream of weights past a tiny x.
//
//   warp 0   TMA producer: cp.async.bulk.tensor loads of a 128 x 64 weight tile and a BN x 64 tile
//            of x per k block into a ring of shared-memory stages (128-byte swizzle), each stage
//            guarded by a full/empty mbarrier pair. Weight tiles depend on no other kernel, so
//            the first ring-full of them is requested before griddepcontrol.wait.
//   warp 1   MMA issuer: allocates tensor memory, and one lane issues four
//            tcgen05.mma.cta_group::1.kind::f16 (K = 16 each) per stage straight from shared
//            memory; tcgen05.commit hands the stage back to the producer and, at the end, the
//            accumulator to the epilogue.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (lane = weight row, column = token), apply the
//            epilogue and write out[token][row]; a warp's 32 lanes write 32 neighbouring columns.
//
// Epilogues: store (bfloat16 or float32); residual (float32 out += result); SwiGLU for a weight
// stacked in blocks of 8 gate rows and 8 up rows (out[T, N / 2] = silu(gate) * up, the partner row
// sits 8 lanes away). With K cut into slices (narrow outputs in decode), every slice's CTA leaves
// its partial tile in scratch and the CTA that arrives last adds them in slice order.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls a CTA sets an abort flag, all its
// roles leave their loops, tensor memory is freed, and *status is set non-zero for the host.
// Any K that is a multiple of 8, any N, any T: tiles that reach past the matrices are zero-filled
// by the TMA unit and their results are not stored.
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;          // weight rows per tile (MMA M)
constexpr int BK = 64;           // k per stage: one 128-byte swizzle atom of bfloat16
constexpr int kThreads = 192;    // producer warp, MMA warp, four epilogue warps

enum Epilogue : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };

struct GemmTcParams {
    void* out;                // EPI_STORE: [T, N]; EPI_RESIDUAL: float [T, N]; EPI_SWIGLU: [T, N / 2]
    const float* bias;        // [N] or null
    float* partials;          // [tiles_m * tiles_n, ksplit, BM * BN] when ksplit > 1
    unsigned int* counters;   // [tiles_m * tiles_n], zero between calls
    int* status;              // set non-zero when a wait gave up
    int T, N, K, ksplit, epilogue, out_f32;
    int vec;                  // rows of out start on 16-byte boundaries: the many-token epilogue may store vectors
    int64_t ldo;
};

// Instruction descriptor of this file's single-CTA products: M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) { return instr_desc_mn(BM, n); }

template <int BN>
struct Smem {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;     // a multiple of 1024 for BN a multiple of 8
};

// One value of the accumulator, after bias, goes out through the chosen epilogue.
template <int BN>
__device__ __forceinline__ void emit(const GemmTcParams& p, float v, int row, int token, int lane) {
    // SwiGLU: lanes 0-7 and 16-23 hold gate rows, the lane 8 further holds the up row of the same output
    if (p.epilogue == EPI_SWIGLU) {
        const float up = __shfl_xor_sync(0xffffffffu, v, 8);
        if ((lane & 8) == 0 && row + 8 < p.N && token < p.T) {
            const float a = v / (1.0f + __expf(-v)) * up;
            const int64_t at = (int64_t)token * p.ldo + (row >> 4) * 8 + (row & 7);
            if (p.out_f32) ((float*)p.out)[at] = a; else ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(a);
        }
        return;
    }
    if (row >= p.N || token >= p.T) return;
    const int64_t at = (int64_t)token * p.ldo + row;
    if (p.epilogue == EPI_RESIDUAL) ((float*)p.out)[at] += v;
    else if (p.out_f32) ((float*)p.out)[at] = v;
    else ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(v);
}

// The many-token kernels keep tokens on the MMA's M side (lane = token, column = weight row), so a thread
// holds neighbouring outputs of one token and stores them as vectors. Sixteen of them, starting at weight
// row f0 (a multiple of 16), leave here through the chosen epilogue.
__device__ __forceinline__ void emit16(const GemmTcParams& p, const uint32_t* r, int token, int f0) {
    if (token >= p.T || f0 >= p.N) return;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
    const bool full = f0 + 16 <= p.N;
    if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (full || f0 + j < p.N) v[j] += __ldg(p.bias + f0 + j);
    }
    if (p.epilogue == EPI_SWIGLU) {   // rows f0..f0+7 are gates, f0+8..f0+15 their up rows; N is a multiple of 16
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = v[j] / (1.0f + __expf(-v[j])) * v[j + 8];
        const int64_t at = (int64_t)token * p.ldo + (f0 >> 1);
        if (p.out_f32) {
            float* o = (float*)p.out + at;
            if (p.vec) {
                ((float4*)o)[0] = make_float4(a[0], a[1], a[2], a[3]);
                ((float4*)o)[1] = make_float4(a[4], a[5], a[6], a[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = a[j];
            }
        } else {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + at;
            if (p.vec) {
                *(uint4*)o = make_uint4(pack_bf16(a[0], a[1]), pack_bf16(a[2], a[3]), pack_bf16(a[4], a[5]), pack_bf16(a[6], a[7]));
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(a[j]);
            }
        }
        return;
    }
    const int64_t at = (int64_t)token * p.ldo + f0;
    if (p.epilogue == EPI_RESIDUAL || p.out_f32) {
        float* o = (float*)p.out + at;
        const bool add = p.epilogue == EPI_RESIDUAL;
        if (p.vec && full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 w = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                if (add) {
                    const float4 old = ((const float4*)o)[q];
                    w.x += old.x; w.y += old.y; w.z += old.z; w.w += old.w;
                }
                ((float4*)o)[q] = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (f0 + j < p.N) o[j] = add ? o[j] + v[j] : v[j];
        }
        return;
    }
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + at;
    if (p.vec && full) {
        ((uint4*)o)[0] = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        ((uint4*)o)[1] = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]), pack_bf16(v[12], v[13]), pack_bf16(v[14], v[15]));
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (f0 + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, (STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 <= 110 * 1024) ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const GemmTcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the stage ring (the swizzle pattern is a function of the address)
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    __shared__ bool is_last;

    constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;           // a power of two >= 32
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = blockIdx.x, tile_n = blockIdx.y, slice = blockIdx.z;
    const int kb_total = (p.K + BK - 1) / BK;
    const int per_slice = (kb_total + p.ksplit - 1) / p.ksplit;
    const int kb0 = slice * per_slice, kb1 = min(kb_total, kb0 + per_slice);
    const int n_kb = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {    // the MMA warp owns tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    pdl_launch_dependents();
    volatile int* abort_p = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const int ahead = min(STAGES, n_kb);
            for (int i = 0; i < ahead; ++i) {        // weights first: they wait for nobody
                const uint32_t full = smem_u32(&bar_full[i]);
                mbar_expect_tx(full, Smem<BN>::kStageBytes);
                tma_load_2d(smem_u32(ring + i * Smem<BN>::kStageBytes), &tmap_w, (kb0 + i) * BK, tile_m * BM, full);
            }
            pdl_wait();                              // x is written by the kernel before this one
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(smem_u32(ring + i * Smem<BN>::kStageBytes + Smem<BN>::kABytes), &tmap_x, (kb0 + i) * BK,
                            tile_n * BN, smem_u32(&bar_full[i]));
            for (int i = ahead; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(smem_u32(&bar_empty[s]), ((i / STAGES) & 1) ^ 1, abort_p)) break;
                const uint32_t full = smem_u32(&bar_full[s]);
                mbar_expect_tx(full, Smem<BN>::kStageBytes);
                tma_load_2d(smem_u32(ring + s * Smem<BN>::kStageBytes), &tmap_w, (kb0 + i) * BK, tile_m * BM, full);
                tma_load_2d(smem_u32(ring + s * Smem<BN>::kStageBytes + Smem<BN>::kABytes), &tmap_x, (kb0 + i) * BK,
                            tile_n * BN, full);
            }
        } else {
            pdl_wait();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        pdl_wait();
        if (lane == 0) {
            const uint32_t acc = tmem_base;
            constexpr uint32_t idesc = instr_desc(BN < 16 ? 16 : BN);
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(smem_u32(&bar_full[s]), (i / STAGES) & 1, abort_p)) break;
                tcgen05_fence_after();
                const uint32_t a_addr = smem_u32(ring + s * Smem<BN>::kStageBytes);
                const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + Smem<BN>::kABytes);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)      // 16 k = 32 bytes further along the swizzled row
                    umma_bf16(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit(smem_u32(&bar_empty[s]));      // the stage is free when these MMAs have read it
            }
            tcgen05_commit(smem_u32(&bar_acc));               // the accumulator is complete
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        pdl_wait();
        const int quarter = warp & 3;                          // the tensor-memory lanes this warp may read
        const int row = tile_m * BM + quarter * 32 + lane;     // weight row = output column
        bool ok = n_kb == 0 || mbar_wait(smem_u32(&bar_acc), 0, abort_p);
        tcgen05_fence_after();
        if (ok) {
            const float b = (p.bias != nullptr && row < p.N && slice == 0) ? p.bias[row] : 0.0f;
            const int64_t tile = (int64_t)tile_m * gridDim.y + tile_n;
            float* mine = p.ksplit > 1 ? p.partials + (tile * p.ksplit + slice) * (int64_t)(BM * BN) : nullptr;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t r[16];
                if (n_kb > 0) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, r);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v = __uint_as_float(r[j]) + b;
                    if (p.ksplit > 1) mine[(c + j) * BM + quarter * 32 + lane] = v;      // [token][row]: coalesced
                    else emit<BN>(p, v, row, tile_n * BN + c + j, lane);
                }
            }
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    if (p.ksplit > 1 && !abort_flag) {
        // the last slice's CTA to arrive adds all slices in slice order
        const int64_t tile = (int64_t)tile_m * gridDim.y + tile_n;
        __threadfence();
        if (threadIdx.x == 0) is_last = atomicAdd(&p.counters[tile], 1u) == (unsigned)p.ksplit - 1;
        __syncthreads();
        if (is_last) {
            __threadfence();
            if (warp >= 2) {
                const int quarter = warp & 3;
                const int row = tile_m * BM + quarter * 32 + lane;
                const float* all = p.partials + tile * p.ksplit * (int64_t)(BM * BN) + quarter * 32 + lane;
                // sixteen tokens at a time: a slice's sixteen loads are in flight together (one after the other, each
                // would wait for L2 on its own), the slices are added in slice order
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    for (int s = 0; s < p.ksplit; ++s) {
                        float t[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) t[j] = __ldcg(all + (int64_t)s * (BM * BN) + (c + j) * BM);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += t[j];
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) emit<BN>(p, v[j], row, tile_n * BN + c + j, lane);
                }
            }
            if (threadIdx.x == 0) p.counters[tile] = 0;
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 1);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Many tokens: a persistent kernel, one CTA an SM, each walking over output tiles (token tile fastest, so
// that the CTAs running at one time share weight tiles in L2). Here the tokens ride the M side (128 a tile)
// and the weight's rows the N side (BN a tile): a thread of the epilogue then holds neighbouring outputs of
// one token and stores 16 bytes at a time. Two accumulators in tensor memory: while the epilogue warps drain
// tile i, the MMA warp already works on tile i + 1. The stage ring runs on across tiles.
template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                          const GemmTcParams p, int tiles_tok, int tiles_f) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;

    constexpr uint32_t kTmemCols = 2 * BN;                       // 256 or 512: a power of two
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (p.K + BK - 1) / BK;
    const int total = tiles_tok * tiles_f;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 4);           // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    pdl_launch_dependents();
    pdl_wait();
    volatile int* abort_p = &abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int t = blockIdx.x; t < total && !*abort_p; t += gridDim.x) {
                const int tile_f = t / tiles_tok, tile_tok = t % tiles_tok;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(smem_u32(&bar_empty[s]), ((it / STAGES) & 1) ^ 1, abort_p)) break;
                    const uint32_t full = smem_u32(&bar_full[s]);
                    mbar_expect_tx(full, Smem<BN>::kStageBytes);
                    tma_load_2d(smem_u32(ring + s * Smem<BN>::kStageBytes), &tmap_x, kb * BK, tile_tok * BM, full);
                    tma_load_2d(smem_u32(ring + s * Smem<BN>::kStageBytes + Smem<BN>::kABytes), &tmap_w, kb * BK,
                                tile_f * BN, full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            int it = 0, lt = 0;
            for (int t = blockIdx.x; t < total && !*abort_p; t += gridDim.x, ++lt) {
                const int buf = lt & 1;
                // the epilogue must have drained this accumulator's previous tile
                if (lt >= 2 && !mbar_wait(smem_u32(&bar_acc_empty[buf]), ((lt >> 1) & 1) ^ 1, abort_p)) break;
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                bool ok = true;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&bar_full[s]), (it / STAGES) & 1, abort_p)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(ring + s * Smem<BN>::kStageBytes);
                    const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + Smem<BN>::kABytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tcgen05_commit(smem_u32(&bar_empty[s]));
                }
                if (!ok) break;
                tcgen05_commit(smem_u32(&bar_acc_full[buf]));
            }
        }
    } else {
        const int quarter = warp & 3;
        int lt = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++lt) {
            const int tile_f = t / tiles_tok, tile_tok = t % tiles_tok, buf = lt & 1;
            if (!mbar_wait(smem_u32(&bar_acc_full[buf]), (lt >> 1) & 1, abort_p)) break;
            tcgen05_fence_after();
            const int token = tile_tok * BM + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                emit16(p, r, token, tile_f * BN + c);
                emit16(p, r + 16, token, tile_f * BN + c + 16);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 1);
}

// ---- CTA pairs (cta_group::2) ---------------------------------------------------------------------------
// Two CTAs of a cluster, on neighbouring SMs, work on one 256 x 256 output tile: each loads 128 of its
// tokens and 128 of its weight rows per k block (32 KB instead of the 48 KB a lone CTA loads for a 128 x 256
// tile: a third less traffic from L2, and fewer TMA rows, per flop), the leader's MMA thread issues
// tcgen05.mma.cta_group::2 with M = 256, which reads both CTAs' shared memory and writes rows 0-127 of the
// accumulator to the leader's tensor memory and rows 128-255 to its peer's. Barriers: both producers' loads
// complete on the leader's full barrier; tcgen05.commit with multicast hands a stage back to both producers
// and the accumulator to both CTAs' epilogue warps; the epilogue warps of both CTAs arrive on the leader's
// accumulator-empty barrier. No load is multicast.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// The shared::cluster address of `addr` (a shared::cta address here) in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// A load into this CTA's shared memory whose bytes are counted on a barrier that may be the peer's.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
// Arrives, once the MMAs issued so far are complete, on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Instruction descriptor of the pair's MMA: M = 256 over both CTAs, N = 256.
__host__ __device__ constexpr uint32_t instr_desc_pair() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

constexpr int kPairTile = 256;                               // weight rows and tokens of a pair's tile
constexpr int kPairStageBytes = 2 * BM * BK * 2;             // per CTA: 128 weight rows and 128 tokens, 64 k each

template <int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const GemmTcParams p, int tiles_tok, int tiles_f) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bar_full[STAGES];       // used in the leader only
    __shared__ __align__(8) uint64_t bar_empty[STAGES];      // one set per CTA, signalled by the leader's commits
    __shared__ __align__(8) uint64_t bar_acc_full[2];        // one set per CTA
    __shared__ __align__(8) uint64_t bar_acc_empty[2];       // used in the leader only: 8 epilogue warps arrive
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;

    constexpr uint32_t kTmemCols = 512;                      // two accumulators of 256 columns
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int n_kb = (p.K + BK - 1) / BK;
    const int total = tiles_tok * tiles_f;
    const int first = (int)cluster_id_x(), step = (int)cluster_count_x();

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                      // the peer's barriers exist before anything signals them
    tcgen05_fence_after();
    pdl_launch_dependents();
    pdl_wait();
    volatile int* abort_p = &abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int t = first; t < total && !*abort_p; t += step) {
                const int tile_f = t / tiles_tok, tile_tok = t % tiles_tok;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait_cluster(smem_u32(&bar_empty[s]), ((it / STAGES) & 1) ^ 1, abort_p)) break;
                    if (leader) mbar_expect_tx(smem_u32(&bar_full[s]), 2 * kPairStageBytes);
                    const uint32_t full = map_to_rank(smem_u32(&bar_full[s]), 0);
                    const uint32_t dst = smem_u32(ring + s * kPairStageBytes);
                    tma_load_2d_pair(dst, &tmap_x, kb * BK, tile_tok * kPairTile + (int)rank * BM, full);
                    tma_load_2d_pair(dst + BM * BK * 2, &tmap_w, kb * BK, tile_f * kPairTile + (int)rank * BM, full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = instr_desc_pair();
            int it = 0, lt = 0;
            for (int t = first; t < total && !*abort_p; t += step, ++lt) {
                const int buf = lt & 1;
                // both CTAs' epilogue warps must have drained this accumulator's previous tile
                if (lt >= 2 && !mbar_wait_cluster(smem_u32(&bar_acc_empty[buf]), ((lt >> 1) & 1) ^ 1, abort_p)) break;
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * kPairTile);
                bool ok = true;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_cluster(smem_u32(&bar_full[s]), (it / STAGES) & 1, abort_p)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(ring + s * kPairStageBytes);
                    const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16_pair(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tcgen05_commit_pair(smem_u32(&bar_empty[s]));
                }
                if (!ok) break;
                tcgen05_commit_pair(smem_u32(&bar_acc_full[buf]));
            }
        }
    } else {
        const int quarter = warp & 3;
        int lt = 0;
        for (int t = first; t < total; t += step, ++lt) {
            const int tile_f = t / tiles_tok, tile_tok = t % tiles_tok, buf = lt & 1;
            if (!mbar_wait_cluster(smem_u32(&bar_acc_full[buf]), (lt >> 1) & 1, abort_p)) break;
            tcgen05_fence_after();
            const int token = tile_tok * kPairTile + (int)rank * BM + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < kPairTile; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kPairTile + c), r);
                emit16(p, r, token, tile_f * kPairTile + c);
                emit16(p, r + 16, token, tile_f * kPairTile + c + 16);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&bar_acc_empty[buf]), 0));
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    cluster_sync_all();                                      // neither CTA frees or leaves while its peer still works
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 1);
}

template <int BN, int STAGES>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcParams& p, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * Smem<BN>::kStageBytes + 1024;
    static bool opted = false;
    if (!opted) {
        cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        opted = true;
    }
    const dim3 grid(ceil_div_i(p.N, BM), ceil_div_i(p.T, BN), p.ksplit);
    return xs_launch(gemm_tc_kernel<BN, STAGES>, grid, dim3(kThreads), smem, stream, mw, mx, p) == cudaSuccess ? 0 : -1;
}

template <int BN, int STAGES>
int launch_persistent(const CUtensorMap& mx, const CUtensorMap& mw, const GemmTcParams& p, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * Smem<BN>::kStageBytes + 1024;
    static bool opted = false;
    static int sms = 0;
    if (!opted) {
        cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        opted = true;
    }
    const int tiles_tok = ceil_div_i(p.T, BM), tiles_f = ceil_div_i(p.N, BN);
    const int grid = tiles_tok * tiles_f < sms ? tiles_tok * tiles_f : sms;
    return xs_launch(gemm_tc_persistent_kernel<BN, STAGES>, dim3(grid), dim3(kThreads), smem, stream, mx, mw, p, tiles_tok,
                     tiles_f) == cudaSuccess ? 0 : -1;
}

int g_pair = 1;   // CTA pairs for more than 128 tokens (xs_gemm_tc_set_pair)
int g_few_deep = 0;   // few tokens: 1 = a deep ring and one CTA an SM; 0 = four stages and two CTAs an SM

template <int STAGES>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const GemmTcParams& p, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * kPairStageBytes + 1024;
    static bool opted = false;
    static int max_pairs = 0;
    if (!opted) {
        cudaFuncSetAttribute(gemm_tc_pair_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        // how many pairs can run at one time: SMs pair up inside a GPC only
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(2 * (sms / 2));
        probe.blockDim = dim3(kThreads);
        probe.dynamicSmemBytes = smem;
        cudaLaunchAttribute a[1];
        a[0].id = cudaLaunchAttributeClusterDimension;
        a[0].val.clusterDim.x = 2; a[0].val.clusterDim.y = 1; a[0].val.clusterDim.z = 1;
        probe.attrs = a;
        probe.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_pair_kernel<STAGES>, &probe) != cudaSuccess || clusters < 1)
            clusters = sms / 2;
        max_pairs = clusters < sms / 2 ? clusters : sms / 2;
        cudaGetLastError();
        opted = true;
    }
    const int tiles_tok = ceil_div_i(p.T, kPairTile), tiles_f = ceil_div_i(p.N, kPairTile);
    const int pairs = tiles_tok * tiles_f < max_pairs ? tiles_tok * tiles_f : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_xs_pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<STAGES>, mx, mw, p, tiles_tok, tiles_f) == cudaSuccess ? 0 : -1;
}

}  // namespace

XS_API void xs_gemm_tc_set_pair(int on) { g_pair = on ? 1 : 0; }
XS_API void xs_gemm_tc_set_few_deep(int on) { g_few_deep = on ? 1 : 0; }

XS_API int xs_gemm_tc_supports(int T, int N, int K, int64_t ldx, int64_t ldw) {
    return T >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && encode_fn() != nullptr;
}

// The token tile the kernel uses for T tokens.
XS_API int xs_gemm_tc_tile_n(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256; }

XS_API int64_t xs_gemm_tc_scratch_bytes(int T, int N, int ksplit) {
    if (ksplit <= 1) return 0;
    const int bn = xs_gemm_tc_tile_n(T);
    const int64_t tiles = (int64_t)ceil_div_i(N, BM) * ceil_div_i(T, bn);
    return tiles * ksplit * BM * bn * (int64_t)sizeof(float) + 65536;
}

// epilogue: 0 store (out_dtype), 1 residual (out is float32 [T, N], += result), 2 SwiGLU (out is [T, N / 2]).
// ksplit > 1: scratch of xs_gemm_tc_scratch_bytes; its last 64 KiB are counters that are zero between calls.
// status: one device int that the kernel sets non-zero if a wait inside it gave up (the result is then invalid).
XS_API int xs_gemm_tc(const void* x, const void* w, const float* bias, void* out, int out_dtype, int epilogue, int T, int N,
                      int K, int64_t ldx, int64_t ldw, int64_t ldo, int ksplit, void* scratch, int64_t scratch_bytes,
                      int* status, cudaStream_t stream) {
    if (T == 0 || N == 0) return 0;
    XS_REQUIRE(xs_gemm_tc_supports(T, N, K, ldx, ldw), "gemm (tcgen05): T %d, N %d, K %d, strides %lld, %lld not supported", T,
               N, K, (long long)ldx, (long long)ldw);
    XS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm (tcgen05): operands must be 16-byte aligned");
    XS_REQUIRE(epilogue >= 0 && epilogue <= 2 && status != nullptr && out != nullptr, "gemm (tcgen05): bad arguments");
    XS_REQUIRE(epilogue != EPI_SWIGLU || N % 16 == 0, "gemm (tcgen05): the fused activation needs N %% 16 == 0");
    XS_REQUIRE(epilogue != EPI_RESIDUAL || out_dtype == XS_F32, "gemm (tcgen05): the residual is float32");
    XS_REQUIRE(ksplit >= 1 && ksplit <= 64, "gemm (tcgen05): %d K slices", ksplit);
    const int bn = xs_gemm_tc_tile_n(T);
    GemmTcParams p;
    p.out = out;
    p.bias = bias;
    p.partials = nullptr;
    p.counters = nullptr;
    p.status = status;
    p.T = T; p.N = N; p.K = K; p.ksplit = ksplit; p.epilogue = epilogue; p.out_f32 = out_dtype == XS_F32;
    p.ldo = ldo;
    p.vec = 0;
    if (ksplit > 1) {
        const int64_t need = xs_gemm_tc_scratch_bytes(T, N, ksplit);
        const int64_t tiles = (int64_t)ceil_div_i(N, BM) * ceil_div_i(T, bn);
        XS_REQUIRE(scratch != nullptr && scratch_bytes >= need && (uintptr_t)scratch % 16 == 0 && tiles * 4 <= 65536,
                   "gemm (tcgen05): %lld bytes of scratch needed for %d K slices, %lld given", (long long)need, ksplit,
                   (long long)scratch_bytes);
        p.partials = (float*)scratch;
        p.counters = (unsigned int*)((char*)scratch + scratch_bytes - 65536);
    }
    alignas(64) CUtensorMap mw, mx;
    int rc;
    if (T <= 64) {
        // few tokens: the weight's rows on the M side, the tokens a narrow N
        XS_REQUIRE(make_map(&mw, w, N, K, ldw, BM), "gemm (tcgen05): the weight's tensor map could not be made");
        XS_REQUIRE(make_map(&mx, x, T, K, ldx, bn), "gemm (tcgen05): the input's tensor map could not be made");
        if (g_few_deep) {
            switch (bn) {
                case 16: rc = launch<16, 8>(mw, mx, p, stream); break;
                case 32: rc = launch<32, 8>(mw, mx, p, stream); break;
                default: rc = launch<64, 6>(mw, mx, p, stream); break;
            }
        } else {
            switch (bn) {
                case 16: rc = launch<16, 5>(mw, mx, p, stream); break;
                case 32: rc = launch<32, 5>(mw, mx, p, stream); break;
                default: rc = launch<64, 4>(mw, mx, p, stream); break;
            }
        }
    } else {
        // many tokens: the tokens on the M side, 128 or 256 weight rows on the N side; pairs of CTAs beyond 128 tokens
        XS_REQUIRE(ksplit == 1, "gemm (tcgen05): K slices are for at most 64 tokens");
        const int esz = p.out_f32 ? 4 : 2;
        p.vec = ((uintptr_t)out % 16 == 0) && ((ldo * esz) % 16 == 0);
        const bool pair = T > 128 && g_pair;
        const int box_w = (pair || N <= 128) ? 128 : 256;
        XS_REQUIRE(make_map(&mx, x, T, K, ldx, BM), "gemm (tcgen05): the input's tensor map could not be made");
        XS_REQUIRE(make_map(&mw, w, N, K, ldw, box_w), "gemm (tcgen05): the weight's tensor map could not be made");
        if (pair) rc = launch_pair<6>(mx, mw, p, stream);
        else if (box_w == 128) rc = launch_persistent<128, 6>(mx, mw, p, stream);
        else rc = launch_persistent<256, 4>(mx, mw, p, stream);
    }
    XS_REQUIRE(rc == 0, "gemm (tcgen05): launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}
