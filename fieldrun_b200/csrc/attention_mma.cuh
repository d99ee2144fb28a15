// Device code of the tensor-core attention over the paged cache for bfloat16 models: one kernel for steps in which every
// sequence brings one token (keys split over blocks, partial results merged in a fixed order) and one for
// steps that bring many tokens per sequence (causal, blockwise with an online softmax).
//
// The formula is the reference's (src/minimax.rs:270-281): s = q.k * scale over the visible keys,
// p = softmax(s), out = p V, query head h reading kv head h / (heads / kv_heads).  Scores, the running
// maximum and sum, and both accumulators are float32; only the operands of the two products are bfloat16.
//
// Both kernels work on tiles of 16 rows x 64 keys (one cache page) held in registers.  Operands go from
// global memory straight into mma.sync fragments with 16-byte loads: a product over k does not depend on
// the order of k, so each thread takes 8 neighbouring elements of k for two MMAs instead of the scattered
// pairs of the fragment layout, on both operands alike.  Values lie transposed within a page
// ([head_dim][64 keys]), which makes the keys of P @ V neighbours in memory too.
#pragma once

#include "common.cuh"

#define ATT_CHUNK 256          // keys per block of the one-token kernel: 4 warps x 1 page

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of 16 rows: lane = 4 g + t holds rows g and g + 8.
template <int HD>
struct RowTile {
    uint4 q[HD / 32][2];       // [32 dims][row g | row g+8]: dims 32 s + 8 t .. + 7
    float o[HD / 8][4];        // [8 dims]: (row g, dims 8 n + 2t, +1), (row g+8, same dims)
    float m[2], l[2];          // running maximum (in units of log2) and sum of rows g and g + 8
};

template <int HD>
__device__ __forceinline__ void tile_init(RowTile<HD>& st) {
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) st.o[n][e] = 0.f;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
}

// Where a page's operands are read from: global memory (the page itself) ...
template <int HD>
struct GlobalPage {
    const bf16* k_page;      // [64][HD]
    const bf16* vt_page;     // [HD][64]
    // 8 dims 32 step + 8 t .. of key `key`
    __device__ __forceinline__ uint4 k(int key, int step, int t) const {
        return __ldg(reinterpret_cast<const uint4*>(k_page + (size_t)key * HD) + step * 4 + t);
    }
    // 8 keys 32 m + 8 t .. of dim `dim`
    __device__ __forceinline__ uint4 v(int dim, int m, int t) const {
        return __ldg(reinterpret_cast<const uint4*>(vt_page + (size_t)dim * FRB_PAGE) + m * 4 + t);
    }
};

// ... or a copy of the page in shared memory, whose 16-byte chunks are swizzled so that the eight lanes of
// a quarter warp (two rows, four chunks each) fall into different banks: chunk ^= (row & 1) << 2, for the
// chunks that lie in whole groups of eight.
template <int CHUNKS_PER_ROW>
__device__ __forceinline__ int swizzled(int chunk, int row) {
    return chunk < (CHUNKS_PER_ROW & ~7) ? chunk ^ ((row & 1) << 2) : chunk;
}

template <int HD>
struct SharedPage {
    const uint4* k_tile;     // [64][HD / 8] chunks
    const uint4* vt_tile;    // [HD][8] chunks
    __device__ __forceinline__ uint4 k(int key, int step, int t) const {
        return k_tile[key * (HD / 8) + swizzled<HD / 8>(step * 4 + t, key)];
    }
    __device__ __forceinline__ uint4 v(int dim, int m, int t) const {
        return vt_tile[dim * 8 + swizzled<8>(m * 4 + t, dim)];
    }
};

// Adds one page of 64 keys to the tile.  key_base: position of the page's first key; row r sees keys
// lo[r] <= j <= hi[r].  scale2 = softmax scale * log2(e).
template <int HD, typename Page>
__device__ __forceinline__ void tile_page(RowTile<HD>& st, const Page& page, int key_base, const int (&lo)[2],
                                          const int (&hi)[2], float scale2, int g, int t) {
    float s[8][4];
    // scores: column block 4 m + u, column c = 2 t' + d of it stands for key 32 m + 8 t' + 2 u + d
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int key_local = 32 * m + 8 * (g >> 1) + 2 * u + (g & 1);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int step = 0; step < HD / 32; ++step) {
                const uint4 kb = page.k(key_local, step, t);
                mma_bf16(acc, st.q[step][0].x, st.q[step][1].x, st.q[step][0].y, st.q[step][1].y, kb.x, kb.y);
                mma_bf16(acc, st.q[step][0].z, st.q[step][1].z, st.q[step][0].w, st.q[step][1].w, kb.z, kb.w);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) s[4 * m + u][e] = acc[e];
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const int key = key_base + 32 * m + 8 * t + 2 * u + (e & 1);
                const float v = (key >= lo[r] && key <= hi[r]) ? s[4 * m + u][e] * scale2 : -INFINITY;
                s[4 * m + u][e] = v;
                mx[r] = fmaxf(mx[r], v);
            }
    float corr[2], sum[2] = {0.f, 0.f}, m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(st.m[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;       // a row that has seen no key yet
        corr[r] = exp2f(st.m[r] - m_use[r]);
        st.m[r] = m_new;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pv = exp2f(s[j][e] - m_use[e >> 1]);
            s[j][e] = pv;
            sum[e >> 1] += pv;
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        st.l[r] = st.l[r] * corr[r] + sum[r];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        st.o[n][0] *= corr[0]; st.o[n][1] *= corr[0];
        st.o[n][2] *= corr[1]; st.o[n][3] *= corr[1];
    }
    // out += P V: the thread's 8 keys 32 m + 8 t .. + 7 are one 16-byte run of a transposed value row
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        const uint32_t a0 = pack_bf16(s[4 * m][0], s[4 * m][1]), a1 = pack_bf16(s[4 * m][2], s[4 * m][3]);
        const uint32_t a2 = pack_bf16(s[4 * m + 1][0], s[4 * m + 1][1]), a3 = pack_bf16(s[4 * m + 1][2], s[4 * m + 1][3]);
        const uint32_t b0 = pack_bf16(s[4 * m + 2][0], s[4 * m + 2][1]), b1 = pack_bf16(s[4 * m + 2][2], s[4 * m + 2][3]);
        const uint32_t b2 = pack_bf16(s[4 * m + 3][0], s[4 * m + 3][1]), b3 = pack_bf16(s[4 * m + 3][2], s[4 * m + 3][3]);
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            const uint4 vb = page.v(8 * n + g, m, t);
            mma_bf16(st.o[n], a0, a1, a2, a3, vb.x, vb.y);
            mma_bf16(st.o[n], b0, b1, b2, b3, vb.z, vb.w);
        }
    }
}

template <int HD>
__device__ __forceinline__ void load_q_row(RowTile<HD>& st, int half, const bf16* __restrict__ row, int t) {
#pragma unroll
    for (int step = 0; step < HD / 32; ++step)
        st.q[step][half] = row ? __ldg(reinterpret_cast<const uint4*>(row + 32 * step) + t) : make_uint4(0, 0, 0, 0);
}

// ----------------------------------------------------------------------------- one token per sequence

struct DecodeAttnParams {
    const bf16* q;             // [B, nh, HD]
    const bf16* k_pages;       // [pages, nkv, 64, HD]
    const bf16* v_pages;       // [pages, nkv, HD, 64]
    const int* page_table;     // [slots, max_pages]
    const int* seq_pos;        // [B] position of the sequence's token
    const int* seq_slot;       // [B]
    float* part_o;             // [B, nh, max_chunks, HD]
    float* part_ml;            // [B, nh, max_chunks, 2]
    bf16* out;                 // [B, nh * HD]
    float scale2;
    int window, max_pages, num_heads, num_kv_heads, max_chunks;
    int* status;               // null, or a word that gets FRB_STATUS_TOO_LONG when a sequence has more chunks than max_chunks
};

#define FRB_STATUS_TOO_LONG 5

// grid (chunk, kv head, sequence), 4 warps.  Rows of the tile are the query heads of the kv head's group.
// Each warp takes one page of the chunk: scores, softmax within the page, then P V in two halves of the
// head size so that few accumulators are alive at a time (more blocks per SM, more loads in flight); the
// four warps' results are combined through shared memory.
template <int HD>
__global__ void __launch_bounds__(128, 4) attention_decode_mma_kernel(DecodeAttnParams p) {
    after_previous_kernel();
    __shared__ float sm_o[4][16][HD + 8];
    __shared__ float sm_m[4][16], sm_l[4][16];
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int group = p.num_heads / p.num_kv_heads;
    const int pos = p.seq_pos[b];
    const int hi_key = pos, lo_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    if (chunk * ATT_CHUNK > hi_key || (chunk + 1) * ATT_CHUNK <= lo_key) return;      // the merge skips these chunks

    const int page_index = chunk * (ATT_CHUNK / FRB_PAGE) + warp;
    const int key_base = page_index * FRB_PAGE;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
    if (key_base <= hi_key && key_base + FRB_PAGE > lo_key) {
        const int page = p.page_table[(size_t)p.seq_slot[b] * p.max_pages + page_index];
        const size_t at = ((size_t)page * p.num_kv_heads + kvh) * FRB_PAGE * HD;
        const GlobalPage<HD> operands = {p.k_pages + at, p.v_pages + at};
        float s[8][4];
        {
            const bf16* q_base = p.q + ((size_t)b * p.num_heads + (size_t)kvh * group) * HD;
            const bf16* q0 = g < group ? q_base + (size_t)g * HD : nullptr;
            const bf16* q1 = g + 8 < group ? q_base + (size_t)(g + 8) * HD : nullptr;
            uint4 q[HD / 32][2];
#pragma unroll
            for (int step = 0; step < HD / 32; ++step) {
                q[step][0] = q0 ? __ldg(reinterpret_cast<const uint4*>(q0 + 32 * step) + t) : make_uint4(0, 0, 0, 0);
                q[step][1] = q1 ? __ldg(reinterpret_cast<const uint4*>(q1 + 32 * step) + t) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int key_local = 32 * m + 8 * (g >> 1) + 2 * u + (g & 1);
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int step = 0; step < HD / 32; ++step) {
                        const uint4 kb = operands.k(key_local, step, t);
                        mma_bf16(acc, q[step][0].x, q[step][1].x, q[step][0].y, q[step][1].y, kb.x, kb.y);
                        mma_bf16(acc, q[step][0].z, q[step][1].z, q[step][0].w, q[step][1].w, kb.z, kb.w);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key_base + 32 * m + 8 * t + 2 * u + (e & 1);
                        const float v = (key >= lo_key && key <= hi_key) ? acc[e] * p.scale2 : -INFINITY;
                        s[4 * m + u][e] = v;
                        row_max[e >> 1] = fmaxf(row_max[e >> 1], v);
                    }
                }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            row_max[r] = fmaxf(row_max[r], __shfl_xor_sync(0xffffffffu, row_max[r], 1));
            row_max[r] = fmaxf(row_max[r], __shfl_xor_sync(0xffffffffu, row_max[r], 2));
        }
        // the page holds at least one visible key, and every row sees the same keys: the maxima are finite
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[j][e] - row_max[e >> 1]);
                s[j][e] = pv;
                row_sum[e >> 1] += pv;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
            row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
        }
        uint32_t pa[2][4], pb[2][4];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            pa[m][0] = pack_bf16(s[4 * m][0], s[4 * m][1]);         pa[m][1] = pack_bf16(s[4 * m][2], s[4 * m][3]);
            pa[m][2] = pack_bf16(s[4 * m + 1][0], s[4 * m + 1][1]); pa[m][3] = pack_bf16(s[4 * m + 1][2], s[4 * m + 1][3]);
            pb[m][0] = pack_bf16(s[4 * m + 2][0], s[4 * m + 2][1]); pb[m][1] = pack_bf16(s[4 * m + 2][2], s[4 * m + 2][3]);
            pb[m][2] = pack_bf16(s[4 * m + 3][0], s[4 * m + 3][1]); pb[m][3] = pack_bf16(s[4 * m + 3][2], s[4 * m + 3][3]);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float o[HD / 16][4];
#pragma unroll
            for (int n = 0; n < HD / 16; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int n = 0; n < HD / 16; ++n) {
                    const uint4 vb = operands.v(8 * (half * (HD / 16) + n) + g, m, t);
                    mma_bf16(o[n], pa[m][0], pa[m][1], pa[m][2], pa[m][3], vb.x, vb.y);
                    mma_bf16(o[n], pb[m][0], pb[m][1], pb[m][2], pb[m][3], vb.z, vb.w);
                }
#pragma unroll
            for (int n = 0; n < HD / 16; ++n) {
                const int d = 8 * (half * (HD / 16) + n) + 2 * t;
                *reinterpret_cast<float2*>(&sm_o[warp][g][d]) = make_float2(o[n][0], o[n][1]);
                *reinterpret_cast<float2*>(&sm_o[warp][g + 8][d]) = make_float2(o[n][2], o[n][3]);
            }
        }
    }
    if (t == 0) {
        sm_m[warp][g] = row_max[0]; sm_l[warp][g] = row_sum[0];
        sm_m[warp][g + 8] = row_max[1]; sm_l[warp][g + 8] = row_sum[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += 128) {
        const int r = idx / HD, d = idx - r * HD;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) top = fmaxf(top, sm_m[w][r]);
        float sum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            if (sm_l[w][r] > 0.f) {                             // a warp whose page holds no visible key wrote nothing
                const float f = exp2f(sm_m[w][r] - top);
                sum += sm_l[w][r] * f;
                acc += sm_o[w][r][d] * f;
            }
        }
        const size_t row = ((size_t)b * p.num_heads + (size_t)kvh * group + r) * p.max_chunks + chunk;
        p.part_o[row * HD + d] = acc;
        if (d == 0) { p.part_ml[row * 2] = top; p.part_ml[row * 2 + 1] = sum; }
    }
}

// Element d of the merged output of one (sequence, head) from the partial results first..last (maximum and sum in
// part_ml, unnormalised output in part_o), first to last.  Eight results at a time, all of their loads asked for
// before the first is used: in a plain loop over the results each load waited for the one before it, which was most of
// the merge's time.
template <int HD>
__device__ __forceinline__ float merged_element(const float* __restrict__ part_ml, const float* __restrict__ part_o, size_t row0,
                                                int first, int last, int d) {
    constexpr int AT_ONCE = 8;
    float top = -INFINITY, sum = 0.f, acc = 0.f;
    for (int c0 = first; c0 <= last; c0 += AT_ONCE) {
        float2 ml[AT_ONCE];
        float o[AT_ONCE];
#pragma unroll
        for (int u = 0; u < AT_ONCE; ++u) {
            const int c = min(c0 + u, last);
            ml[u] = *reinterpret_cast<const float2*>(part_ml + (row0 + c) * 2);
            o[u] = part_o[(row0 + c) * HD + d];
        }
        float group_top = top;
#pragma unroll
        for (int u = 0; u < AT_ONCE; ++u)
            if (c0 + u <= last) group_top = fmaxf(group_top, ml[u].x);
        // what was summed so far follows the new maximum (nothing was summed before the first group)
        const float keep = top == -INFINITY ? 0.f : exp2f(top - group_top);
        sum *= keep;
        acc *= keep;
        top = group_top;
#pragma unroll
        for (int u = 0; u < AT_ONCE; ++u)
            if (c0 + u <= last) {
                const float f = exp2f(ml[u].x - top);
                sum += ml[u].y * f;
                acc += o[u] * f;
            }
    }
    return acc / sum;
}

// grid (head, sequence): merges the chunks of one (sequence, head), first chunk to last.
template <int HD>
__global__ void __launch_bounds__(HD) attention_decode_merge_kernel(DecodeAttnParams p) {
    after_previous_kernel();
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const int pos = p.seq_pos[b];
    const int lo_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    // never beyond the partial results the launch has room for, whatever the position says (the caller's
    // max_chunks covers the longest sequence; a smaller one must not make this read another row's results)
    const int last = min(pos / ATT_CHUNK, p.max_chunks - 1), first = min(lo_key / ATT_CHUNK, last);
    if (pos / ATT_CHUNK >= p.max_chunks && p.status && d == 0) atomicExch(p.status, FRB_STATUS_TOO_LONG);   // keys were left out
    const size_t row0 = ((size_t)b * p.num_heads + head) * p.max_chunks;
    p.out[((size_t)b * p.num_heads + head) * HD + d] = __float2bfloat16_rn(merged_element<HD>(p.part_ml, p.part_o, row0, first, last, d));
}

// Checks the sizes and launches the one-token kernel and its merge.  `what` names the caller in errors.
static inline int launch_attention_decode(const char* what, const void* q, const void* k_pages, const void* v_pages,
                                          const int* page_table, int max_pages, const int* seq_pos, const int* seq_slot,
                                          float* part_o, float* part_ml, void* out, int num_seqs, int num_heads,
                                          int num_kv_heads, int head_dim, float scale, int window, int max_chunks,
                                          cudaStream_t stream, int* status = nullptr) {
    if (num_seqs == 0) return 0;
    const int group = num_kv_heads > 0 ? num_heads / num_kv_heads : 0;
    FRB_CHECK_ARG(num_kv_heads > 0 && num_heads % num_kv_heads == 0 && group <= 16,
                  "%s: %d heads over %d kv heads (groups of at most 16)", what, num_heads, num_kv_heads);
    FRB_CHECK_ARG(head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128,
                  "%s: head_dim %d is not 32, 64, 96 or 128", what, head_dim);
    FRB_CHECK_ARG(num_seqs <= 65535 && num_kv_heads <= 65535, "%s: %d sequences exceed the grid", what, num_seqs);
    DecodeAttnParams p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages; p.page_table = page_table;
    p.seq_pos = seq_pos; p.seq_slot = seq_slot; p.part_o = part_o; p.part_ml = part_ml; p.out = (bf16*)out;
    p.scale2 = scale * 1.4426950408889634f; p.window = window; p.max_pages = max_pages; p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads; p.max_chunks = max_chunks; p.status = status;
    dim3 grid(max_chunks, num_kv_heads, num_seqs), merge_grid(num_heads, num_seqs);
#define FRB_LAUNCH_DECODE(HD)                                                       \
    launch_dependent(attention_decode_mma_kernel<HD>, dim3(grid), dim3(128), 0, stream, p);                   \
    launch_dependent(attention_decode_merge_kernel<HD>, dim3(merge_grid), dim3(HD), 0, stream, p)
    if (head_dim == 32) { FRB_LAUNCH_DECODE(32); } else if (head_dim == 64) { FRB_LAUNCH_DECODE(64); }
    else if (head_dim == 96) { FRB_LAUNCH_DECODE(96); } else { FRB_LAUNCH_DECODE(128); }
#undef FRB_LAUNCH_DECODE
    FRB_RETURN_LAUNCH(what);
}
