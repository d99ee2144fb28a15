// Attention over the paged cache, any head size up to 256 and any group size, float32 arithmetic.
// It is the whole attention of the float32 path and the fallback of the bfloat16 path for shapes that
// the tensor-core kernels refuse.
//
// Per query head h with kv = h / (nh / nkv): s_j = (q . K_j) * scale for the keys the query may see
// (j <= its position, and j > position - window when a window is set), p = exp(s - max) / sum,
// out = sum_j p_j V_j  (src/minimax.rs:270-281).  Keys that are hidden get weight 0 exactly, which is what
// the reference's -1e30 amounts to after the exponential.
#include "common.cuh"

struct AttnParams {
    const void* q;            // [T, nh, hd]
    const void* k_pages;      // [pages, nkv, PAGE, hd]
    const void* v_pages;      // [pages, nkv, hd, PAGE]: values lie transposed within a page
    const int* page_table;    // [slots, max_pages]
    const int* tok_pos;       // [T]
    const int* tok_slot;      // [T]
    void* out;                // [T, nh * hd]
    float scale;
    int window;               // 0: every earlier key
    int max_pages, num_heads, num_kv_heads, head_dim;
};

#define KEY_BLOCK 32

// grid (token, kv head); one warp per query head of the group, warps share the staged K/V block.
template <typename T>
__global__ void attention_generic_kernel(AttnParams p) {
    extern __shared__ float sm[];
    const int hd = p.head_dim;
    float* k_tile = sm;                                  // [KEY_BLOCK][hd + 1]
    float* v_tile = k_tile + KEY_BLOCK * (hd + 1);       // [KEY_BLOCK][hd]
    float* q_rows = v_tile + KEY_BLOCK * hd;             // [warps][hd]
    const int t = blockIdx.x, g = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int group = p.num_heads / p.num_kv_heads;
    const int pos = p.tok_pos[t];
    const int hi = pos;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int* table = p.page_table + (size_t)p.tok_slot[t] * p.max_pages;
    const T* q = (const T*)p.q;
    const T* k_pages = (const T*)p.k_pages;
    const T* v_pages = (const T*)p.v_pages;
    T* out = (T*)p.out;

    for (int hbase = 0; hbase < group; hbase += nwarps) {
        const int hl = hbase + warp;
        const bool active = hl < group;
        const int head = g * group + hl;
        if (active)
            for (int d = lane; d < hd; d += 32) q_rows[warp * hd + d] = to_f32<T>(q[((size_t)t * p.num_heads + head) * hd + d]);
        float m = -INFINITY, l = 0.f;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;

        for (int j0 = (lo / KEY_BLOCK) * KEY_BLOCK; j0 <= hi; j0 += KEY_BLOCK) {
            __syncthreads();
            const int page = table[j0 / FRB_PAGE];
            const size_t head_base = ((size_t)page * p.num_kv_heads + g) * FRB_PAGE * hd;
            const int in_page = j0 % FRB_PAGE;
            for (int i = threadIdx.x; i < KEY_BLOCK * hd; i += blockDim.x) {
                const int r = i / hd, d = i - r * hd;
                const bool valid = (j0 + r >= lo) && (j0 + r <= hi);
                k_tile[r * (hd + 1) + d] = valid ? to_f32<T>(k_pages[head_base + (size_t)(in_page + r) * hd + d]) : 0.f;
            }
            for (int i = threadIdx.x; i < KEY_BLOCK * hd; i += blockDim.x) {
                const int d = i / KEY_BLOCK, r = i - d * KEY_BLOCK;          // keys of one dim are neighbours in memory
                const bool valid = (j0 + r >= lo) && (j0 + r <= hi);
                v_tile[r * hd + d] = valid ? to_f32<T>(v_pages[head_base + (size_t)d * FRB_PAGE + in_page + r]) : 0.f;
            }
            __syncthreads();
            if (active) {
                const int j = j0 + lane;
                const bool valid = (j >= lo) && (j <= hi);
                float s = 0.f;
                const float* qr = q_rows + warp * hd;
                const float* kr = k_tile + lane * (hd + 1);
                for (int d = 0; d < hd; ++d) s += qr[d] * kr[d];
                s = valid ? s * p.scale : -INFINITY;
                const float m_new = fmaxf(m, warp_max(s));
                const float corr = expf(m - m_new);
                const float pj = valid ? expf(s - m_new) : 0.f;
                l = l * corr + warp_sum(pj);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] *= corr;
                for (int kk = 0; kk < KEY_BLOCK; ++kk) {
                    const float pk = __shfl_sync(0xffffffffu, pj, kk);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int d = lane + 32 * i;
                        if (d < hd) acc[i] += pk * v_tile[kk * hd + d];
                    }
                }
                m = m_new;
            }
        }
        if (active) {
            const float inv = 1.0f / l;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) out[((size_t)t * p.num_heads + head) * hd + d] = from_f32<T>(acc[i] * inv);
            }
        }
    }
}

FRB_API int frb_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                  const int* page_table, int max_pages, const int* tok_pos, const int* tok_slot,
                                  void* out, int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                  float scale, int window, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(head_dim >= 1 && head_dim <= 256, "attention: head_dim %d is outside 1..256", head_dim);
    FRB_CHECK_ARG(num_kv_heads >= 1 && num_heads % num_kv_heads == 0, "attention: %d heads are not a multiple of %d kv heads",
                  num_heads, num_kv_heads);
    FRB_CHECK_ARG(num_kv_heads <= 65535, "attention: %d kv heads exceed the grid", num_kv_heads);
    AttnParams p;
    p.q = q; p.k_pages = k_pages; p.v_pages = v_pages; p.page_table = page_table; p.tok_pos = tok_pos;
    p.tok_slot = tok_slot; p.out = out; p.scale = scale; p.window = window; p.max_pages = max_pages;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
    const int group = num_heads / num_kv_heads;
    const int nwarps = group < 8 ? group : 8;
    const size_t smem = ((size_t)KEY_BLOCK * (head_dim + 1) + (size_t)KEY_BLOCK * head_dim + (size_t)nwarps * head_dim) * sizeof(float);
    dim3 grid(num_tokens, num_kv_heads);
    FRB_DISPATCH_DTYPE(dtype, T, {
        auto kernel = attention_generic_kernel<T>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<grid, 32 * nwarps, smem, stream>>>(p);
    });
    FRB_RETURN_LAUNCH("attention_generic");
}
