// Shared helpers of the sm_100a kernels: element types, error reporting, reductions.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and the
// stream to launch on, allocates nothing, and returns 0 or a negative code after
// recording a message that xs_last_error() returns. Sizes a kernel cannot take are
// refused here on the host, never computed wrongly.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define XS_API extern "C" __attribute__((visibility("default")))

enum XsDType : int { XS_F32 = 0, XS_BF16 = 1 };

void xs_set_error(const char* fmt, ...);

#define XS_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            xs_set_error(__VA_ARGS__);   \
            return -1;                   \
        }                                \
    } while (0)

#define XS_LAUNCH_CHECK(name)                                                      \
    do {                                                                           \
        cudaError_t e_ = cudaGetLastError();                                       \
        if (e_ != cudaSuccess) {                                                   \
            xs_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));   \
            return -2;                                                             \
        }                                                                          \
    } while (0)

// Dispatch on one element type code.
#define XS_DISPATCH_DTYPE(code, T, ...)                         \
    do {                                                        \
        if ((code) == XS_F32) {                                 \
            using T = float;                                    \
            __VA_ARGS__;                                        \
        } else if ((code) == XS_BF16) {                         \
            using T = __nv_bfloat16;                            \
            __VA_ARGS__;                                        \
        } else {                                                \
            xs_set_error("unknown element type code %d", (int)(code)); \
            return -1;                                          \
        }                                                       \
    } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. Every thread gets the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();   // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float t = lane < warps ? scratch[lane] : 0.0f;
    return warp_sum(t);
}

static inline int ceil_div_i(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// ---- programmatic dependent launch ------------------------------------------------------------
// A decode step is a chain of some 150 short kernels, each waiting for the one before it. Launched
// with the attribute below, a kernel may start while its predecessor is still draining: it runs up
// to pdl_wait() (address arithmetic, and in the few-row product the first weight loads, which
// depend on nothing), and only there waits until the predecessor has completed and its writes are
// visible. Rules every kernel here keeps: nothing that another kernel of the step writes is read,
// and nothing at all is written to global memory, before pdl_wait(). Without the attribute both
// calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::); }

extern int g_xs_pdl;   // 1: launches carry the attribute (xs_set_pdl)

// `carveout` >= 0: this launch prefers that much of an SM's memory as shared memory (per cent of the most), the rest as L1
// cache; -1 leaves the choice to the driver. It matters beyond the kernel itself: a neighbour of the step that overlaps this
// kernel on an SM (programmatic dependent launch) runs under the same split, and the few-row products want their L1.
template <typename... KArgs, typename... Args>
inline cudaError_t xs_launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int carveout,
                                Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (g_xs_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (carveout >= 0) {
        attr[n].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
        attr[n].val.sharedMemCarveout = (unsigned int)carveout;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid cut into thread-block clusters of `cluster` CTAs (which must divide the grid).
template <typename... KArgs, typename... Args>
inline cudaError_t xs_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (g_xs_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t xs_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    return xs_launch_ex(kernel, grid, block, smem, stream, -1, args...);
}
