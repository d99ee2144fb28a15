// Entry points of the tensor-core attention (bfloat16): steps of one token per sequence, and steps of many.
// The kernels are in attention_mma.cuh.
#include "attention_mma.cuh"

FRB_API int frb_attention_decode_mma(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                     int max_pages, const int* seq_pos, const int* seq_slot, float* part_o, float* part_ml,
                                     void* out, int num_seqs, int num_heads, int num_kv_heads, int head_dim, float scale,
                                     int window, int max_chunks, int* status, cudaStream_t stream) {
    return launch_attention_decode("attention_decode_mma", q, k_pages, v_pages, page_table, max_pages, seq_pos, seq_slot,
                                   part_o, part_ml, out, num_seqs, num_heads, num_kv_heads, head_dim, scale, window,
                                   max_chunks, stream, status);
}

// ----------------------------------------------------------------------------- many tokens per sequence

struct PrefillAttnParams {
    const bf16* q;             // [T, nh, HD]
    const bf16* k_pages;
    const bf16* v_pages;
    const int* page_table;
    const int* tile_seq;       // [tiles] sequence of the tile
    const int* tile_q0;        // [tiles] first row of the tile among its sequence's new tokens
    const int* seq_slot;       // [B]
    const int* seq_start;      // [B] position of the sequence's first new token
    const int* seq_q_len;      // [B]
    const int* cu_q_len;       // [B + 1]
    bf16* out;                 // [T, nh * HD]
    float scale2;
    int window, max_pages, num_heads, num_kv_heads;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Starts the copy of one page's keys and transposed values into a stage of shared memory (swizzled chunks).
template <int HD>
__device__ __forceinline__ void stage_page(uint4* k_tile, uint4* vt_tile, const bf16* __restrict__ k_page,
                                           const bf16* __restrict__ vt_page) {
    constexpr int CHUNKS = FRB_PAGE * HD / 8;           // 16-byte chunks of K, and as many of V
    for (int c = threadIdx.x; c < CHUNKS; c += blockDim.x) {
        const int key = c / (HD / 8), chunk = c % (HD / 8);
        cp_async16(k_tile + key * (HD / 8) + swizzled<HD / 8>(chunk, key), reinterpret_cast<const uint4*>(k_page) + c);
        const int dim = c >> 3, vchunk = c & 7;
        cp_async16(vt_tile + dim * 8 + swizzled<8>(vchunk, dim), reinterpret_cast<const uint4*>(vt_page) + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// grid (tile of 16 queries, kv head).  The warps of a block take the query heads of the kv head's group:
// they need the same keys and values, which the block copies page by page into two stages of shared memory
// with cp.async, the next page on its way while the current one is multiplied.
template <int HD, int MAX_WARPS>
__global__ void __launch_bounds__(MAX_WARPS * 32, MAX_WARPS <= 6 ? 2 : 1) attention_prefill_mma_kernel(PrefillAttnParams p) {
    extern __shared__ uint4 stages[];                   // 2 x (K tile, V^T tile), FRB_PAGE * HD / 8 chunks each
    constexpr int TILE = FRB_PAGE * HD / 8;
    const int tile = blockIdx.x, kvh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, g = lane >> 2, t = lane & 3;
    const int group = p.num_heads / p.num_kv_heads;
    const int b = p.tile_seq[tile], q0 = p.tile_q0[tile];
    const int q_len = p.seq_q_len[b], start = p.seq_start[b], tok0 = p.cu_q_len[b] + q0;
    const int* table = p.page_table + (size_t)p.seq_slot[b] * p.max_pages;
    int lo[2], hi[2];
    bool valid[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        valid[r] = q0 + row < q_len;
        hi[r] = valid[r] ? start + q0 + row : -1;
        lo[r] = (valid[r] && p.window > 0) ? max(0, hi[r] - p.window + 1) : 0;
    }
    const int last_key = start + min(q0 + 15, q_len - 1);
    const int first_key = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;
    const int first_page = first_key / FRB_PAGE, last_page = last_key / FRB_PAGE;
    for (int hbase = 0; hbase < group; hbase += nwarps) {
        const int hl = hbase + warp;
        const bool active = hl < group;
        const int head = kvh * group + (active ? hl : 0);
        RowTile<HD> st;
        tile_init(st);
#pragma unroll
        for (int r = 0; r < 2; ++r)
            load_q_row(st, r, (active && valid[r]) ? p.q + ((size_t)(tok0 + g + 8 * r) * p.num_heads + head) * HD : nullptr, t);
        {
            const size_t at = ((size_t)table[first_page] * p.num_kv_heads + kvh) * FRB_PAGE * HD;
            stage_page<HD>(stages, stages + TILE, p.k_pages + at, p.v_pages + at);
        }
        for (int page_index = first_page; page_index <= last_page; ++page_index) {
            const int cur = (page_index - first_page) & 1;
            if (page_index < last_page) {
                const size_t at = ((size_t)table[page_index + 1] * p.num_kv_heads + kvh) * FRB_PAGE * HD;
                stage_page<HD>(stages + (cur ^ 1) * 2 * TILE, stages + (cur ^ 1) * 2 * TILE + TILE, p.k_pages + at, p.v_pages + at);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            if (active) {
                const SharedPage<HD> page = {stages + cur * 2 * TILE, stages + cur * 2 * TILE + TILE};
                tile_page(st, page, page_index * FRB_PAGE, lo, hi, p.scale2, g, t);
            }
            __syncthreads();                            // the stage is free for the page after the next
        }
        if (active) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                if (!valid[r]) continue;
                const float inv = 1.0f / st.l[r];
                bf16* dst = p.out + ((size_t)(tok0 + g + 8 * r) * p.num_heads + head) * HD;
#pragma unroll
                for (int n = 0; n < HD / 8; ++n)
                    *reinterpret_cast<uint32_t*>(dst + 8 * n + 2 * t) = pack_bf16(st.o[n][2 * r] * inv, st.o[n][2 * r + 1] * inv);
            }
        }
    }
}

FRB_API int frb_attention_prefill_mma(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                      int max_pages, const int* tile_seq, const int* tile_q0, int num_tiles,
                                      const int* seq_slot, const int* seq_start, const int* seq_q_len, const int* cu_q_len,
                                      void* out, int num_heads, int num_kv_heads, int head_dim, float scale, int window,
                                      cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    FRB_CHECK_ARG(num_kv_heads > 0 && num_heads % num_kv_heads == 0, "attention: %d heads over %d kv heads", num_heads, num_kv_heads);
    FRB_CHECK_ARG(head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128,
                  "attention: head_dim %d is not 32, 64, 96 or 128", head_dim);
    FRB_CHECK_ARG(num_kv_heads <= 65535, "attention: %d kv heads exceed the grid", num_kv_heads);
    PrefillAttnParams p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages; p.page_table = page_table;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.seq_slot = seq_slot; p.seq_start = seq_start; p.seq_q_len = seq_q_len;
    p.cu_q_len = cu_q_len; p.out = (bf16*)out; p.scale2 = scale * 1.4426950408889634f; p.window = window;
    p.max_pages = max_pages; p.num_heads = num_heads; p.num_kv_heads = num_kv_heads;
    const int group = num_heads / num_kv_heads;
    const int nwarps = group < 8 ? group : 8;
    dim3 grid(num_tiles, num_kv_heads);
    const size_t smem = (size_t)4 * FRB_PAGE * head_dim * sizeof(bf16);           // two stages of K and V^T
    // groups of up to 6 heads: blocks of at most 192 threads, held to two per SM; larger groups: 256 threads
#define LAUNCH(HD)                                                                                                  \
    if (nwarps <= 6) {                                                                                              \
        if (smem > 48 * 1024)                                                                                       \
            cudaFuncSetAttribute(attention_prefill_mma_kernel<HD, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        attention_prefill_mma_kernel<HD, 6><<<grid, 32 * nwarps, smem, stream>>>(p);                                \
    } else {                                                                                                        \
        if (smem > 48 * 1024)                                                                                       \
            cudaFuncSetAttribute(attention_prefill_mma_kernel<HD, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        attention_prefill_mma_kernel<HD, 8><<<grid, 32 * nwarps, smem, stream>>>(p);                                \
    }
    if (head_dim == 32) { LAUNCH(32); } else if (head_dim == 64) { LAUNCH(64); } else if (head_dim == 96) { LAUNCH(96); } else { LAUNCH(128); }
#undef LAUNCH
    FRB_RETURN_LAUNCH("attention_prefill_mma");
}
