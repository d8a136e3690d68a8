/* Allocation-free all-gather entry point.
 *
 * This entry point has no counterpart in the reference; it exists for callers that are not
 * allowed to allocate device memory: code running where the memory pool is owned by someone else
 * (an inference server that hands this library a fixed arena, a plugin inside another framework's
 * allocator), or where cudaMalloc's implicit device synchronisation is unacceptable in the middle
 * of a serving loop. The regular kr_all_gather_sm() needs zeroed arrival counters that either the
 * caller allocates or the library allocates on first use; this variant keeps them, and a status
 * word, in a fixed array compiled into the library.
 *
 * Limits and rules:
 *   - world_size * splits <= KR_NOALLOC_MAX_CHUNKS; larger requests are rejected with an error.
 *   - The scratch (KR_NOALLOC_SCRATCH_BYTES per GPU) lives in every GPU that loads the library,
 *     for the life of the process.
 *   - The first call on each device looks up the scratch address (a host-side query, no
 *     allocation). Make that first call outside of any stream capture.
 *   - All calls on one device share the scratch. The counters are cleared on `stream` at the start
 *     of every call, so two calls whose kernels can overlap on the GPU (different streams) race;
 *     issue them on one stream or order them with events.
 *   - No cudaMalloc / cudaFree / allocating library routine is called. Inputs and outputs —
 *     including the pointer tables `bufs` and `pads`, `output`, `progress` and the optional
 *     `status` word — are the caller's memory.
 */
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

#define KR_NOALLOC_MAX_CHUNKS 1024
#define KR_NOALLOC_SCRATCH_BYTES (256 + 4 * KR_NOALLOC_MAX_CHUNKS)

#ifdef __cplusplus
extern "C" {
#endif

/* output[world_size * numel] = concatenation over ranks r of bufs[r][buf_off .. buf_off + numel)
 * (numel counts 2-byte elements); progress[src * splits + split] becomes 1 when that chunk has
 * landed. Same semantics and arguments as kr_all_gather_sm(), minus its `counters` argument,
 * plus `status`: an optional device word (zero on entry) that receives a non-zero code if a
 * bounded wait gave up; pass NULL to use a word inside the library's scratch.
 * Returns 0 on success; on failure kr_last_error() describes the problem. */
int kr_all_gather_sm_noalloc(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank,
                             int world_size, void* output, uint32_t* progress, int splits,
                             unsigned long long numel, int max_blocks, uint32_t pad_base, uint32_t* status,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
