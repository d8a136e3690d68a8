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
 *   - All calls on one device share the scratch. The counters (and, for calls that pass
 *     status == NULL, the built-in status word) are cleared on `stream` at the start of every
 *     call, so two calls whose kernels can overlap on the GPU (different streams) race; issue them
 *     on one stream or order them with events.
 *   - `stream` must belong to the current device (the scratch address is per device); a stream of
 *     another device is rejected.
 *   - Failure reporting. Every device-side wait has a deadline (kr_noalloc_set_timeout_ms; default:
 *     the library-wide setting). When one expires the kernel writes a non-zero code to the status
 *     word, copies nothing more and returns; the host call has long returned 0 by then. A status
 *     word the caller passes must be zero on entry and is the caller's to read and to clear. With
 *     status == NULL the code goes to the built-in word: read it with kr_noalloc_read_status()
 *     after the call you want to check — the next call with status == NULL starts by clearing it,
 *     so a past timeout neither lingers nor makes later calls give up.
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

/* Synchronises `stream`, then stores the built-in status word of the current device in *word
 * (0 = no wait gave up); clear != 0 also zeroes it. Allocates nothing. */
int kr_noalloc_read_status(cudaStream_t stream, uint32_t* word, int clear);

/* Deadline, in milliseconds, of the device-side waits of kr_all_gather_sm_noalloc; 0 restores the
 * default (the value of kr_set_timeout_ms for the current device if that was ever called, else
 * KRAKEN_SYNC_TIMEOUT_MS, else 4000 ms). Allocates nothing. */
int kr_noalloc_set_timeout_ms(double ms);

#ifdef __cplusplus
}
#endif
