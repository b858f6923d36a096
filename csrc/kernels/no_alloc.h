// Allocation-free decode attention entry point.
//
// This entry point has no counterpart in the reference framework.  It exists for
// callers that are not allowed to allocate device memory at the moment they run
// attention: code that executes inside a region where cudaMalloc / cudaFree are
// forbidden or would synchronise the device (a real-time serving loop with a
// frozen memory budget, a plugin running inside another framework's allocator
// arena, a process whose memory was sized up front and must not grow).  Such a
// caller cannot provide the split-KV scratch buffer that nkb_paged_attn_decode
// needs when num_splits > 1, so this variant keeps that scratch inside the
// library: a fixed 16 MiB device array that every GPU which loads the library
// holds until the process exits.
//
//   * Inputs and outputs are still the caller's buffers; only the scratch is ours.
//   * The call rejects (returns NKB_NOALLOC_TOO_LARGE and prints one line to
//     stderr) any problem whose scratch need
//         16384 + batch * nkv * num_splits * (16 * head_dim + 32) floats
//     exceeds NKB_NOALLOC_SCRATCH_FLOATS, or that has more than 16384
//     (sequence, kv head) pairs.  num_splits == 1 needs no scratch.
//   * The first call on each device looks up the device address of the array
//     (and of a private status word).  Make that first call before starting any
//     stream capture on that device.  The look-up is guarded by a mutex, so two
//     host threads may both make "the first call".
//   * All calls share the one array, and it keeps whatever the previous call
//     left in it.  The array begins with the arrival counters of the split
//     merge, which must count from zero: each call clears the counters it uses
//     with a memset on its stream before the kernel (the partial results behind
//     them need no clearing, every slot that the merge reads is written earlier
//     in the same call).  Two calls that may run at the same time on the GPU
//     (different streams) would overwrite each other's counters and partial
//     results: serialise them.
//   * A wait inside the kernel that gives up (after one second) reports into a
//     status word of this entry point's own, read with nkb_noalloc_status();
//     nkb_status() covers the other entry points only.
//   * The function calls no cudaMalloc, cudaFree or allocating library routine.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NKB_NOALLOC_SCRATCH_FLOATS (4ll * 1024 * 1024) /* 16 MiB */
#define NKB_NOALLOC_TOO_LARGE (-10)   /* scratch need exceeds the built-in array */
#define NKB_NOALLOC_SETUP_FAILED (-11) /* cudaGetSymbolAddress / device query failed */

// Same arguments and semantics as nkb_paged_attn_decode (api.h) without the
// scratch pointer.  Returns 0 on a successful launch, a negative code for a
// rejected argument, or a positive CUDA error code.
int nkb_paged_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                  const int* context_lens, void* out, int batch, int q_len, int nq, int nkv,
                                  int head_dim, int block_size, int num_blocks, int max_blocks_per_seq, float scale,
                                  int window, const float* sinks, int num_splits, void* stream);

// Reads (reset != 0: and clears) the status word of the allocation-free entry point on the current
// device: 0, or the code of a bounded wait that gave up (low byte) with the CTA index above it.
// Synchronises the device.  Negative: the set-up failed.
int nkb_noalloc_status(int reset);

#ifdef __cplusplus
}
#endif
