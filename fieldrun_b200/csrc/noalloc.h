/* fieldrun_b200: an attention entry point that allocates nothing.
 *
 * This entry point has no counterpart in the reference (jascal/fieldrun is a CPU program and never manages
 * device memory); it exists for callers of this library who may not allocate device memory themselves.
 *
 * Who that is.  Some programs that embed these kernels must not call cudaMalloc, cudaFree or any routine
 * that allocates behind their back (torch's caching allocator included) at the time they run a step:
 *   - a serving loop that took all the device memory it will ever own at start-up and hands the rest to
 *     another tenant, so that a later allocation can fail or evict someone;
 *   - a latency-critical loop, because cudaMalloc and cudaFree synchronise the whole device;
 *   - code that runs between cudaStreamBeginCapture and cudaStreamEndCapture, where an allocation is an error.
 * The ordinary one-token attention (frb_attention_decode_mma) needs scratch memory for the partial results
 * of its key chunks and expects the caller to bring it.  This variant brings its own: a fixed array that
 * is part of the library's image on the device.
 *
 * What it costs.  FRB_NOALLOC_SCRATCH_FLOATS floats (8 MiB) of device memory on every GPU that loads the
 * library, from load until the process exits, whether or not this entry point is ever called.
 *
 * Limits.  The partial results need num_seqs * num_heads * max_chunks * (head_dim + 2) floats; a call that
 * needs more than FRB_NOALLOC_SCRATCH_FLOATS is refused with an error (nothing is launched).  Inputs and
 * outputs are still the caller's.
 *
 * First call.  The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 * with that device current).  Make that first call outside any stream capture.  No call allocates.
 *
 * Sharing.  Every call on a device uses the same array, and the array keeps what the last call left in it.
 * Nothing in it has to start at zero: a call writes every entry it later reads.  Two calls that overlap
 * on the GPU (different streams, no ordering between them) race on the array and give wrong results; order
 * them on one stream or with events.
 */
#ifndef FIELDRUN_B200_NOALLOC_H
#define FIELDRUN_B200_NOALLOC_H

#include <cuda_runtime.h>

#define FRB_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

/* One-token attention over the paged cache (bfloat16), same arguments and results as
 * frb_attention_decode_mma without the two scratch pointers.  Returns 0, or non-zero after leaving a message
 * for frb_last_error().
 *   q           [num_seqs, num_heads, head_dim] bfloat16
 *   k_pages     [pages, num_kv_heads, 64, head_dim] bfloat16
 *   v_pages     [pages, num_kv_heads, head_dim, 64] bfloat16
 *   page_table  [slots, max_pages] int32
 *   seq_pos     [num_seqs] int32, position of each sequence's token;  seq_slot [num_seqs] int32
 *   out         [num_seqs, num_heads * head_dim] bfloat16
 *   max_chunks  ceil((largest position + 1) / 256) or more
 */
int frb_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                 int max_pages, const int* seq_pos, const int* seq_slot, void* out, int num_seqs,
                                 int num_heads, int num_kv_heads, int head_dim, float scale, int window, int max_chunks,
                                 cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif
