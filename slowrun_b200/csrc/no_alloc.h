/* Allocation-free entry point of the slowrun_b200 kernel library.
 *
 * This function has no counterpart in the reference project; it exists for callers of the library that are not
 * allowed to allocate device memory at the point where they need the Muon post-processing step:
 *   - code running inside another framework's allocator hook or gradient-ready callback, where calling back into
 *     that framework's caching allocator (or cudaMalloc, which synchronises the device) is forbidden;
 *   - processes that hand out all device memory at start-up and keep no head-room for later cudaMalloc calls.
 *
 * It computes exactly what sr_muon_post computes (NorMuon variance reduction of an orthogonalised stack X[n, r, c]:
 * second-moment update of S in place, and the scaled bf16 update U), but takes no work arrays: they live in a
 * fixed 2 MiB device array inside the library, resident on every GPU that loads it until the process exits.
 *
 * Limits and rules
 *   - n * max(r, c) <= sr_muon_post_noalloc_max_elems() (262144); otherwise -8 is returned and nothing runs.
 *   - c must be a multiple of 4 (-2 otherwise). Other negative codes: -5 launch failure, -9 the device address of
 *     the internal array could not be obtained, -10 unsupported device ordinal.
 *   - The first call on a device performs a one-time lookup of the array's device address; issue it before any
 *     stream capture begins on that device.
 *   - The stream must belong to the device that is current when the function is called; the first call for a device
 *     must not race with another thread's first call for the same device.
 *   - Calls share the internal array. Calls whose kernels may overlap on the GPU must be ordered by the caller
 *     (same stream, or events); unordered concurrent calls race.
 *   - The caller still owns and passes X (bf16, read), S (fp32 state, updated) and U (bf16, written).
 *   - Nothing on this path calls cudaMalloc, cudaFree or an allocating library routine.
 */
#pragma once
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

long sr_muon_post_noalloc_max_elems(void);

int sr_muon_post_noalloc(const void* X /* bf16 [n, r, c] */, float* S /* fp32 [n, max-dim side] */,
                         void* U /* bf16 [n, r, c] out */, int n, int r, int c, float beta2, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
