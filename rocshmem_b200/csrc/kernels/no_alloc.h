/* Allocation-free entry point of librocshmem_b200.so. It has no counterpart in the reference.
 *
 * Who needs it: callers that are not allowed to allocate device memory at the point where they
 * need the MoE expert layout. Typical cases are a serving engine that hands the whole GPU memory to
 * its own pool at start-up and forbids cudaMalloc afterwards, a plug-in running inside such a
 * process, and code on a latency path where an allocation (which may synchronise the device) is
 * unacceptable. The regular entry point, ep_expert_layout(), expects the caller to bring a scratch
 * array of per-expert cursors; this variant keeps that scratch in a fixed array inside the library.
 *
 * What it computes (same result as ep_expert_layout): given the metadata records and the row
 * bookkeeping written by the MoE dispatch, it groups the received rows by local expert:
 *   offsets[e] .. offsets[e + 1]   positions that belong to local expert e (experts_per_rank + 1 ints)
 *   row_index[pos]                 received row at that position
 *   pair_k[pos]                    which of the row's top-k entries selected expert e
 * The order of positions inside one expert's range is unspecified.
 *
 * Limits: experts_per_rank <= ROCSHMEM_B200_NOALLOC_MAX_EXPERTS (1024), n_ranks <= 64, top_k <= 8.
 * Larger values are refused with ROCSHMEM_B200_NOALLOC_TOO_LARGE and a message on stderr; nothing is
 * launched in that case. The scratch is 4 KiB of device memory per GPU that has loaded the library,
 * held until the process exits.
 *
 * Rules of use:
 *   - The first call on each device looks up the device address of the scratch array (with that
 *     device current) and caches it. Make that first call outside any stream capture. The cached
 *     address does not survive cudaDeviceReset(): do not reset a device after its first call.
 *   - experts_per_rank must be the value the dispatch was configured with. Pairs whose expert index is
 *     not below experts_per_rank are left out of the layout.
 *   - All calls on a device share the one scratch array. The kernels clear what they need at the
 *     start of every call, so calls that follow each other on one stream are fine; calls that may
 *     overlap on the GPU (different streams, no dependency) race on the scratch and must be avoided.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, here or in the kernels.
 *   - All pointers are device pointers supplied by the caller; `stream` is a cudaStream_t.
 *
 * Returns 0 on success, a positive cudaError_t value if a CUDA call failed, or one of the negative
 * codes below.
 */
#ifndef ROCSHMEM_B200_NO_ALLOC_H_
#define ROCSHMEM_B200_NO_ALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define ROCSHMEM_B200_NOALLOC_MAX_EXPERTS 1024
#define ROCSHMEM_B200_NOALLOC_TOO_LARGE (-2)
#define ROCSHMEM_B200_NOALLOC_BAD_ARGUMENT (-3)

int rocshmem_b200_expert_layout_noalloc(const int *recv_meta, const int *recv_info, int n_ranks,
                                        int experts_per_rank, int top_k, int *offsets, int *row_index,
                                        int *pair_k, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* ROCSHMEM_B200_NO_ALLOC_H_ */
