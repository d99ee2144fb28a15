// One-token attention that brings its own scratch memory: see noalloc.h for who needs it and what it costs.
// The kernels are the ones of attention_mma.cuh; only the home of the partial results differs.
#include "attention_mma.cuh"
#include "noalloc.h"

// Partial outputs and (maximum, sum) pairs of the key chunks.  It lives in the library's device image.
// In host code this name is only a handle: the address the kernels need comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[FRB_NOALLOC_SCRATCH_FLOATS];

#define FRB_NOALLOC_MAX_DEVICES 64
static float* g_scratch_address[FRB_NOALLOC_MAX_DEVICES];       // per device, looked up at the first call there

extern "C" __attribute__((visibility("default")))
int frb_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                 int max_pages, const int* seq_pos, const int* seq_slot, void* out, int num_seqs,
                                 int num_heads, int num_kv_heads, int head_dim, float scale, int window, int max_chunks,
                                 cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(num_seqs > 0 && num_heads > 0 && max_chunks > 0 && head_dim > 0, "attention_decode_noalloc: sizes must be positive");
    const unsigned long long rows = (unsigned long long)num_seqs * num_heads * max_chunks;
    const unsigned long long need = rows * ((unsigned long long)head_dim + 2);
    FRB_CHECK_ARG(need <= FRB_NOALLOC_SCRATCH_FLOATS,
                  "attention_decode_noalloc: %d sequences x %d heads x %d chunks x (%d + 2) = %llu floats of partial results, "
                  "the built-in scratch holds %u; use frb_attention_decode_mma with scratch of your own",
                  num_seqs, num_heads, max_chunks, head_dim, need, FRB_NOALLOC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    FRB_CHECK_ARG(err == cudaSuccess && device >= 0 && device < FRB_NOALLOC_MAX_DEVICES,
                  "attention_decode_noalloc: no usable current device (%s)", cudaGetErrorString(err));
    if (g_scratch_address[device] == nullptr) {
        float* address = nullptr;
        err = cudaGetSymbolAddress((void**)&address, g_noalloc_scratch);     // the array's address on the current device
        FRB_CHECK_ARG(err == cudaSuccess && address != nullptr, "attention_decode_noalloc: cudaGetSymbolAddress failed: %s",
                      cudaGetErrorString(err));
        g_scratch_address[device] = address;
    }
    float* part_o = g_scratch_address[device];                  // [num_seqs, num_heads, max_chunks, head_dim]
    float* part_ml = part_o + rows * head_dim;                  // [num_seqs, num_heads, max_chunks, 2]
    return launch_attention_decode("attention_decode_noalloc", q, k_pages, v_pages, page_table, max_pages, seq_pos, seq_slot,
                                   part_o, part_ml, out, num_seqs, num_heads, num_kv_heads, head_dim, scale, window, max_chunks,
                                   stream);
}
