/* Allocation-free GLA forward entry point (libtriune_noalloc.so).
 *
 * This entry point has no counterpart in the reference project. It exists for callers that must not allocate
 * device memory while they run: code replaying work inside a serving loop with a fixed memory plan, plugins that
 * are handed a device but no allocator, and hosts where cudaMalloc would synchronise the whole device at a bad
 * moment. The chunked GLA forward needs scratch (per-chunk state contributions, per-chunk decays, the chunk-start
 * states and a status word); here that scratch is a fixed array inside the library, so the call performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Limits and rules
 *   - B * H * (T / 64) <= TRIUNE_NOALLOC_MAX_CHUNKS (512); larger problems are rejected with -2.
 *   - head_dim is 64, T is a positive multiple of 64, tensors are bf16 [B*T, H*64] row-major, 16-byte aligned.
 *   - The scratch array (about 12.3 MB) is part of the library image: every GPU that loads the library holds it
 *     until the process exits.
 *   - The first call on EACH device resolves the device address of that array on that device
 *     (cudaGetSymbolAddress, with the device current) and sets the kernels' shared-memory attributes there. Make
 *     that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents; the entry point clears the words
 *     that must start at zero itself. Two calls that overlap on the GPU (different streams, no ordering) race on
 *     the scratch and give wrong results: order them on one stream or with events.
 */
#ifndef TRIUNE_B200_GLA_NOALLOC_H
#define TRIUNE_B200_GLA_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRIUNE_NOALLOC_MAX_CHUNKS 512

/* out[B*T, H*64] = GLA(q, k, v, g); final_state[B*H, 64, 64] (fp32) receives the state after the last token.
 * init_state may be NULL (zero initial state). gate_logits != 0: g holds raw gate logits (log-sigmoid applied
 * inside). Returns 0 on success, -1 bad argument, -2 problem larger than the built-in scratch, -3 CUDA error
 * (cudaGetLastError() has the detail). The work is enqueued on `stream`; read *status_out after synchronising:
 * 0 means every bounded wait inside the kernels completed. status_out may be NULL; when given it should point to
 * pinned (page-locked) host memory: the status word is copied with cudaMemcpyAsync, and a copy into pageable memory
 * makes the runtime stage it and blocks the calling thread until the stream has drained. */
int triune_gla_forward_noalloc(const void* q, const void* k, const void* v, const void* g, void* out, float* final_state,
                               const float* init_state, int B, int T, int H, int gate_logits, int* status_out,
                               cudaStream_t stream);

/* Bytes of built-in scratch (for documentation / tests). */
unsigned long long triune_gla_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
#endif
