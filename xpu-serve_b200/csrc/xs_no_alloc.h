// An entry point for callers that cannot allocate device memory.
//
// This declaration has no counterpart in the reference project; it exists for this library's own
// users. Split-key attention (xs_attention_mma with splits > 1) needs scratch memory for the
// partial results that its CTAs exchange, and normally the caller passes a buffer. Some callers
// have no way to get one: code that runs inside a CUDA-graph capture or a real-time loop where
// cudaMalloc is forbidden, a plug-in that is handed only the tensors of its operation, or a host
// language binding without an allocator of its own. For them, xs_attention_mma_static keeps the
// scratch in a file-scope device array inside the library.
//
// What to know before using it:
//  * The array is kScratchBytes (8 MiB) of every GPU's memory for as long as the library is
//    loaded on it, whether or not the function is ever called.
//  * A problem whose partial results do not fit (tokens * heads * splits * (head_dim + 2) * 4 bytes
//    > 8 MiB) is refused with an error; nothing is computed.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress).
//    Make that first call outside any stream capture; later calls do no set-up.
//  * All calls share the one array. Calls that may run at the same time on one GPU (different
//    streams, different threads) would overwrite each other's partial results: serialise them.
//  * The array keeps whatever the last call left. The kernels write every word they later read,
//    so nothing needs clearing between calls.
//  * The function itself calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as xs_attention_mma (attention_mma.cu), without `scratch` and
// `scratch_bytes`. Returns 0, or a negative code after recording a message for xs_last_error().
int xs_attention_mma_static(const void* q, const void* pool, const int32_t* page_table, int P,
                            const int32_t* cu_seqlens, const int32_t* kv_lens, const void* gate, int64_t ld_gate,
                            void* out, int T, int n_seqs, int max_q_len, int Hq, int Hkv, int D, int page_size,
                            float scale, int window, int splits, cudaStream_t stream);

// The size of the built-in scratch array in bytes.
int64_t xs_attention_mma_static_capacity(void);

#ifdef __cplusplus
}
#endif
