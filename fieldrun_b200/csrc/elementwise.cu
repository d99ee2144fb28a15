// Row-wise kernels: embedding rows, RMSNorm fused with the residual add that precedes it,
// and the step between the QKV product and attention (full-width Q/K RMSNorm, rotary on the
// first rotary_dim dims of each head, write of K and V into the paged cache).
//
// Formulas follow the reference's CPU code: norm x*rsqrt(mean(x^2)+eps)*w (src/minimax.rs:56-66),
// rotate-half pairs (j, j+half) by pos*inv[j] (src/minimax.rs:69-84, partial form
// src/qwen35moe.rs:121-138), K cached after norm and rotary, V as projected (src/minimax.rs:262-268).
// All statistics and the residual sum are float32.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_error[1024] = "";

void frb_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
}

FRB_API const char* frb_last_error() { return g_error; }

FRB_API int frb_abi_version() { return 3; }

// ----------------------------------------------------------------------------- embedding rows

template <typename WT>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const WT* __restrict__ table, float* __restrict__ out,
                                  int width, int vocab) {
    after_previous_kernel();
    const int t = blockIdx.x;
    int token = tokens[t];
    if (token < 0 || token >= vocab) token = 0;      // ids are checked on the host before any launch
    const WT* row = table + (size_t)token * width;
    float* dst = out + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_f32<WT>(row[i]);
}

// out[t, :] = table[tokens[t], :] widened to float32 (no multiplier, src/minimax.rs:132).
FRB_API int frb_embed_rows(const int* tokens, const void* table, int table_dtype, float* out, int num_tokens,
                           int width, int vocab, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_DISPATCH_DTYPE(table_dtype, WT, {
        launch_dependent(embed_rows_kernel<WT>, dim3(num_tokens), dim3(256), 0, stream, tokens, (const WT*)table, out, width, vocab);
    });
    FRB_RETURN_LAUNCH("embed_rows");
}

// Four neighbouring elements at once.
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned int*>(&lo);
    raw.y = *reinterpret_cast<const unsigned int*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// ----------------------------------------------------------------------------- RMSNorm (+ residual add)

// Rows are one block each.  A step of few rows takes blocks of 1024 threads (the row's latency is the step's);
// a step of many rows takes blocks of 256 (more blocks per SM, less waiting at the block's barriers).
#define NORM_FEW_ROWS 64
#define NORM_MAX_TOP_K 32

// The update of the residual stream may come as the outputs of a token's experts, not yet summed:
// update[src] = sum over ranks r, in rank order, of weights[src, r] * y[row_of_assign[src * k + r]]
// (src/minimax.rs:121-123).
struct ExpertSum {
    const float* y;               // [N, width], null: none
    const float* weights;         // [T, k]
    const int* row_of_assign;     // [T * k]
    int top_k;
};

// One block per output row r.  src = rows ? rows[r] : r.  v = x[src] (+ delta[src]) (+ the experts' sum of
// src); if write_back the sum is stored to x[src] (the residual stream).
// out[r] = v * (1/sqrt(mean(v^2)+eps)) * w, in OutT and, when out32 is given, in float32 as well.
template <typename OutT, typename WT, int NORM_BLOCK, bool VEC>
__global__ void __launch_bounds__(NORM_BLOCK)
rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, ExpertSum experts, const int* __restrict__ rows,
               const WT* __restrict__ weight, float eps, int width, OutT* __restrict__ out, float* __restrict__ out32,
               int write_back) {
    // The norm's weight is nobody's output: it is loaded before the kernel before this one has ended.
    constexpr int EARLY = 2;                                   // groups of four weights a thread holds in registers
    const bool early = VEC && width <= 4 * EARLY * NORM_BLOCK;
    float4 w_early[EARLY];
    let_next_kernel_start();
    if (early) {
#pragma unroll
        for (int u = 0; u < EARLY; ++u) {
            const int i = 4 * (u * NORM_BLOCK + threadIdx.x);
            if (i < width) w_early[u] = load4<WT>(weight + i);
        }
    }
    wait_for_previous_kernel();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    __shared__ float expert_weight[NORM_MAX_TOP_K];
    __shared__ const float* expert_row[NORM_MAX_TOP_K];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * width;
    const float* dr = delta ? delta + (size_t)src * width : nullptr;
    if (experts.y) {                       // the token's weights and rows first, so that the loads below do not wait in turn
        if (threadIdx.x < experts.top_k) {
            const int at = src * experts.top_k + threadIdx.x;
            expert_weight[threadIdx.x] = experts.weights[at];
            expert_row[threadIdx.x] = experts.y + (size_t)experts.row_of_assign[at] * width;
        }
        __syncthreads();
    }
    float ss = 0.f;
    if (VEC) {
        // four elements at a time; a token's expert rows are loaded together, then added in rank order
        for (int i = 4 * threadIdx.x; i < width; i += 4 * NORM_BLOCK) {
            float4 v = *reinterpret_cast<const float4*>(xr + i);
            if (dr) {
                const float4 d = *reinterpret_cast<const float4*>(dr + i);
                v = make_float4(v.x + d.x, v.y + d.y, v.z + d.z, v.w + d.w);
            }
            if (experts.y) {
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int k0 = 0; k0 < experts.top_k; k0 += 8) {
                    float4 part[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (k0 + k < experts.top_k) part[k] = *reinterpret_cast<const float4*>(expert_row[k0 + k] + i);
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (k0 + k < experts.top_k) {
                            const float w = expert_weight[k0 + k];
                            sum = make_float4(sum.x + w * part[k].x, sum.y + w * part[k].y, sum.z + w * part[k].z, sum.w + w * part[k].w);
                        }
                }
                v = make_float4(v.x + sum.x, v.y + sum.y, v.z + sum.z, v.w + sum.w);
            }
            *reinterpret_cast<float4*>(row + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (write_back) *reinterpret_cast<float4*>(xr + i) = v;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += NORM_BLOCK) {
            float v = xr[i];
            if (dr) v += dr[i];
            if (experts.y) {
                float sum = 0.f;
                for (int k = 0; k < experts.top_k; ++k) sum += expert_weight[k] * expert_row[k][i];
                v += sum;
            }
            row[i] = v;
            ss += v * v;
            if (write_back) xr[i] = v;
        }
    }
    ss = block_sum<NORM_BLOCK>(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)width + eps);
    if (early) {
#pragma unroll
        for (int u = 0; u < EARLY; ++u) {
            const int i = 4 * (u * NORM_BLOCK + threadIdx.x);
            if (i < width) {
                const float4 v = *reinterpret_cast<const float4*>(row + i);
                const float4 w = w_early[u];
                const float4 y = make_float4(v.x * rinv * w.x, v.y * rinv * w.y, v.z * rinv * w.z, v.w * rinv * w.w);
                store4<OutT>(out + (size_t)r * width + i, y);
                if (out32) *reinterpret_cast<float4*>(out32 + (size_t)r * width + i) = y;
            }
        }
    } else if (VEC) {
        for (int i = 4 * threadIdx.x; i < width; i += 4 * NORM_BLOCK) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            const float4 w = load4<WT>(weight + i);
            const float4 y = make_float4(v.x * rinv * w.x, v.y * rinv * w.y, v.z * rinv * w.z, v.w * rinv * w.w);
            store4<OutT>(out + (size_t)r * width + i, y);
            if (out32) *reinterpret_cast<float4*>(out32 + (size_t)r * width + i) = y;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += NORM_BLOCK) {
            const float y = row[i] * rinv * to_f32<WT>(weight[i]);
            out[(size_t)r * width + i] = from_f32<OutT>(y);
            if (out32) out32[(size_t)r * width + i] = y;
        }
    }
}

FRB_API int frb_rmsnorm(float* x, const float* delta, const float* expert_y, const float* expert_weights,
                        const int* row_of_assign, int top_k, const int* rows, const void* weight, int weight_dtype,
                        float eps, int num_rows, int width, void* out, int out_dtype, float* out32,
                        int write_back, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(expert_y == nullptr || (top_k >= 1 && top_k <= NORM_MAX_TOP_K), "rmsnorm: %d experts per token exceed %d",
                  top_k, NORM_MAX_TOP_K);
    ExpertSum experts = {expert_y, expert_weights, row_of_assign, top_k};
    const size_t smem = (size_t)width * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "rmsnorm: width %d needs %zu bytes of shared memory, more than 200 KB", width, smem);
    const auto on16 = [](const void* ptr) { return ((uintptr_t)ptr & 15) == 0; };
    const bool by_four = width % 4 == 0 && on16(x) && on16(delta) && on16(expert_y) && on16(out) && on16(out32) && on16(weight);
    FRB_DISPATCH_DTYPE(out_dtype, OutT, FRB_DISPATCH_DTYPE(weight_dtype, WT, {
        // with the experts' outputs to sum (nine rows read per token) the wide block is the faster one at any number of
        // rows: 2,048 rows 72 -> 63 us, 16,384 rows 504 -> 466
        if (num_rows <= NORM_FEW_ROWS || expert_y) {
            auto kernel = by_four ? rmsnorm_kernel<OutT, WT, 1024, true> : rmsnorm_kernel<OutT, WT, 1024, false>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_rows), dim3(1024), smem, stream, x, delta, experts, rows, (const WT*)weight, eps, width,
                             (OutT*)out, out32, write_back);
        } else {
            auto kernel = by_four ? rmsnorm_kernel<OutT, WT, 256, true> : rmsnorm_kernel<OutT, WT, 256, false>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_rows), dim3(256), smem, stream, x, delta, experts, rows, (const WT*)weight, eps, width,
                             (OutT*)out, out32, write_back);
        }
    }));
    FRB_RETURN_LAUNCH("rmsnorm");
}

// ----------------------------------------------------------------------------- Q/K norm + rotary + cache write

struct QkvParams {
    const void* qkv;          // [T, (nh + 2 nkv) * hd], InT
    const void* q_weight;     // [nh*hd] or null: no norm
    const void* k_weight;     // [nkv*hd] or null
    const float* cos_table;   // [positions, rotary_dim/2]
    const float* sin_table;
    const int* tok_pos;       // [T] absolute position
    const int* tok_slot;      // [T] cache slot
    const int* page_table;    // [slots, max_pages]
    void* q_out;              // [T, nh, hd] OutT
    void* k_pages;            // [pages, nkv, PAGE, hd] OutT
    void* v_pages;            // [pages, nkv, hd, PAGE] OutT: values lie transposed within a page
    float eps;
    int num_heads, num_kv_heads, head_dim, rotary_dim, interleaved, max_pages, write_cache, table_positions;
    int num_tokens, v_tiles;  // v_tiles: the grid's first v_tiles blocks write the values, 64 tokens of one kv head each
    int per_head;             // the norm weights are [head_dim] and every head has a statistic of its own
    int tables_final;         // positions, slots and page table were complete before the kernel before this one began
    unsigned head_dim_inverse;   // ceil(2^32 / head_dim): the high word of n times this is n / head_dim for n < 2^24
};

#define QKV_BATCH 8          // elements a thread loads before it uses any of them

// One block per token.  A thread first issues all of its loads (a batch of raw values with their norm
// weights), so that their latencies overlap; the rows then sit in shared memory, Q and K already multiplied
// by their weights, and each thread produces output elements from its own element and its rotation partner.
template <typename InT, typename OutT, typename WT, int NORM_BLOCK>
__global__ void __launch_bounds__(NORM_BLOCK) qkv_prepare_kernel(QkvParams p) {
    after_previous_kernel();
    extern __shared__ float raw[];           // [(nh + 2 nkv) * hd] : Q row, K row, V row; then cos and sin [rotary_dim / 2]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int hd = p.head_dim;
    const int q_width = p.num_heads * hd, k_width = p.num_kv_heads * hd;
    const int qk_width = q_width + k_width, all_width = qk_width + k_width;
    const int half = p.rotary_dim / 2;
    float* s_cos = raw + all_width;
    float* s_sin = s_cos + half;
    float* s_sq = s_sin + half;              // per-head norm only: the squares [qk_width], then 1/rms of every head
    float* s_rinv = s_sq + qk_width;
    const InT* src = (const InT*)p.qkv + (size_t)t * all_width;
    const WT* qw = (const WT*)p.q_weight;
    const WT* kw = (const WT*)p.k_weight;

    const int pos = p.tok_pos[t];
    const int slot = p.tok_slot[t];
    float ssq = 0.f, ssk = 0.f;
    for (int base = 0; base < all_width; base += QKV_BATCH * NORM_BLOCK) {
        float v[QKV_BATCH], w[QKV_BATCH];
#pragma unroll
        for (int u = 0; u < QKV_BATCH; ++u) {
            const int i = base + u * NORM_BLOCK + threadIdx.x;
            v[u] = i < all_width ? to_f32<InT>(src[i]) : 0.f;
            w[u] = 1.f;
            if (i < q_width) { if (qw) w[u] = to_f32<WT>(qw[p.per_head ? i % hd : i]); }
            else if (i < qk_width) { if (kw) w[u] = to_f32<WT>(kw[p.per_head ? (i - q_width) % hd : i - q_width]); }
        }
#pragma unroll
        for (int u = 0; u < QKV_BATCH; ++u) {
            const int i = base + u * NORM_BLOCK + threadIdx.x;
            if (i < all_width) raw[i] = v[u] * w[u];
            if (i < q_width) ssq += v[u] * v[u];
            else if (i < qk_width) ssk += v[u] * v[u];
            if (p.per_head && i < qk_width) s_sq[i] = v[u] * v[u];
        }
    }
    const int table_row = pos < p.table_positions ? pos : p.table_positions - 1;   // positions are checked on the host
    for (int j = threadIdx.x; j < half; j += NORM_BLOCK) {
        s_cos[j] = p.cos_table[(size_t)table_row * half + j];
        s_sin[j] = p.sin_table[(size_t)table_row * half + j];
    }
    const int page = p.write_cache ? p.page_table[(size_t)slot * p.max_pages + pos / FRB_PAGE] : -1;
    const int in_page = pos % FRB_PAGE;
    float rinv_q = 1.f, rinv_k = 1.f;
    if (qw && !p.per_head) rinv_q = 1.0f / sqrtf(block_sum<NORM_BLOCK>(ssq, scratch) / (float)q_width + p.eps);
    if (kw && !p.per_head) rinv_k = 1.0f / sqrtf(block_sum<NORM_BLOCK>(ssk, scratch) / (float)k_width + p.eps);
    __syncthreads();
    if (p.per_head) {
        // one statistic per head (q heads, then k heads): a warp sums a head's squares in a fixed order
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int h = warp; h < p.num_heads + p.num_kv_heads; h += NORM_BLOCK / 32) {
            float ss = 0.f;
            for (int d = lane; d < hd; d += 32) ss += s_sq[h * hd + d];
            ss = warp_sum(ss);
            if (lane == 0) s_rinv[h] = (h < p.num_heads ? qw : kw) ? 1.0f / sqrtf(ss / (float)hd + p.eps) : 1.f;
        }
        __syncthreads();
    }

    for (int i = threadIdx.x; i < qk_width; i += NORM_BLOCK) {
        const bool is_q = i < q_width;
        const float* base = is_q ? raw : raw + q_width;
        const int local = is_q ? i : i - q_width;
        const int head = local / hd, dim = local - head * hd;
        const float rinv = p.per_head ? s_rinv[(is_q ? 0 : p.num_heads) + head] : (is_q ? rinv_q : rinv_k);
        float value = base[local] * rinv;
        if (dim < p.rotary_dim) {
            int j, partner;
            bool first;
            if (p.interleaved) { j = dim >> 1; first = (dim & 1) == 0; partner = first ? local + 1 : local - 1; }
            else { first = dim < half; j = first ? dim : dim - half; partner = first ? local + half : local - half; }
            const float other = base[partner] * rinv;
            const float c = s_cos[j], s = s_sin[j];
            // a' = a c - b s ; b' = b c + a s   (src/minimax.rs:78-81)
            value = first ? value * c - other * s : value * c + other * s;
        }
        if (is_q) {
            ((OutT*)p.q_out)[(size_t)t * q_width + local] = from_f32<OutT>(value);
        } else if (page >= 0) {
            const size_t at = (((size_t)page * p.num_kv_heads + head) * FRB_PAGE + in_page) * hd + dim;
            ((OutT*)p.k_pages)[at] = from_f32<OutT>(value);
        }
    }
    if (page >= 0) {
        const float* vrow = raw + qk_width;
        for (int i = threadIdx.x; i < k_width; i += NORM_BLOCK) {
            const int head = i / hd, dim = i - head * hd;
            const size_t at = (((size_t)page * p.num_kv_heads + head) * hd + dim) * FRB_PAGE + in_page;
            ((OutT*)p.v_pages)[at] = from_f32<OutT>(vrow[i]);
        }
    }
}

#define QKV_VEC_BATCH 4      // groups of four elements a thread loads before it uses any of them
#define QKV_V_TOKENS 64      // tokens whose values one block transposes

// The same work four elements at a time, for head sizes and rotation widths in steps of four (eight for the
// half-split pairing, so that a group's partners are a group too) and rows that start on 16 bytes.
template <typename InT, typename OutT, typename WT, int NORM_BLOCK>
__global__ void __launch_bounds__(NORM_BLOCK) qkv_prepare_vec_kernel(QkvParams p) {
    let_next_kernel_start();
    extern __shared__ __align__(16) float raw[];   // Q row, K row, V row; then cos and sin [rotary_dim / 2]
    __shared__ float scratch[64];
    const int hd = p.head_dim;
    const int q_width = p.num_heads * hd, k_width = p.num_kv_heads * hd;
    const int qk_width = q_width + k_width, all_width = qk_width + k_width;
    int pos_early = 0, slot_early = 0, page_early = -1;
    // the blocks that transpose values come first in the grid: they run longest, and at the grid's end they ran alone
    const int token_block = (int)blockIdx.x - p.v_tiles;
    if (p.tables_final && token_block >= 0) {
        // positions, slots, pages and angles were there before the kernel before this one began
        pos_early = p.tok_pos[token_block];
        slot_early = p.tok_slot[token_block];
        const int table_row = pos_early < p.table_positions ? pos_early : p.table_positions - 1;
        float* s_cos = raw + all_width;
        float* s_sin = s_cos + p.rotary_dim / 2;
        for (int j = threadIdx.x; j < p.rotary_dim / 2; j += NORM_BLOCK) {
            s_cos[j] = p.cos_table[(size_t)table_row * (p.rotary_dim / 2) + j];
            s_sin[j] = p.sin_table[(size_t)table_row * (p.rotary_dim / 2) + j];
        }
        page_early = p.write_cache ? p.page_table[(size_t)slot_early * p.max_pages + pos_early / FRB_PAGE] : -1;
    }
    wait_for_previous_kernel();
    if (token_block < 0) {
        // The values of 64 tokens of one kv head: read along the dimensions, written along the tokens, whose
        // places in a transposed page are neighbours whenever their positions are (a prompt's are).
        __shared__ int s_page[QKV_V_TOKENS], s_place[QKV_V_TOKENS];
        OutT* tile = reinterpret_cast<OutT*>(raw);                       // [hd][QKV_V_TOKENS + 2]
        const int index = blockIdx.x;
        const int h = index % p.num_kv_heads, t0 = (index / p.num_kv_heads) * QKV_V_TOKENS;
        const int count = min(QKV_V_TOKENS, p.num_tokens - t0);
        for (int j = threadIdx.x; j < count; j += NORM_BLOCK) {
            const int pos = p.tok_pos[t0 + j];
            s_page[j] = p.page_table[(size_t)p.tok_slot[t0 + j] * p.max_pages + pos / FRB_PAGE];
            s_place[j] = pos % FRB_PAGE;
        }
        // a warp reads a token's dimensions, then writes a dimension's tokens: no division per element
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int j = warp; j < count; j += NORM_BLOCK / 32) {
            const InT* row = (const InT*)p.qkv + (size_t)(t0 + j) * all_width + qk_width + h * hd;
            for (int d = lane; d < hd; d += 32) tile[d * (QKV_V_TOKENS + 2) + j] = from_f32<OutT>(to_f32<InT>(row[d]));
        }
        __syncthreads();
        for (int d = warp; d < hd; d += NORM_BLOCK / 32) {
            for (int j = lane; j < count; j += 32) {
                const size_t at = (((size_t)s_page[j] * p.num_kv_heads + h) * hd + d) * FRB_PAGE + s_place[j];
                ((OutT*)p.v_pages)[at] = tile[d * (QKV_V_TOKENS + 2) + j];
            }
        }
        return;
    }
    const int t = token_block;
    const int row_width = p.v_tiles ? qk_width : all_width;               // the values are other blocks' work then
    const int half = p.rotary_dim / 2;
    float* s_cos = raw + all_width;
    float* s_sin = s_cos + half;
    const InT* src = (const InT*)p.qkv + (size_t)t * all_width;
    const WT* qw = (const WT*)p.q_weight;
    const WT* kw = (const WT*)p.k_weight;

    const int pos = p.tables_final ? pos_early : p.tok_pos[t];
    const int slot = p.tables_final ? slot_early : p.tok_slot[t];
    float ssq = 0.f, ssk = 0.f;
    for (int base = 0; base < row_width; base += 4 * QKV_VEC_BATCH * NORM_BLOCK) {
        float4 v[QKV_VEC_BATCH], w[QKV_VEC_BATCH];
#pragma unroll
        for (int u = 0; u < QKV_VEC_BATCH; ++u) {
            const int i = base + 4 * (u * NORM_BLOCK + threadIdx.x);
            v[u] = i < row_width ? load4<InT>(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            w[u] = make_float4(1.f, 1.f, 1.f, 1.f);
            if (i < q_width) { if (qw) w[u] = load4<WT>(qw + i); }
            else if (i < qk_width) { if (kw) w[u] = load4<WT>(kw + i - q_width); }
        }
#pragma unroll
        for (int u = 0; u < QKV_VEC_BATCH; ++u) {
            const int i = base + 4 * (u * NORM_BLOCK + threadIdx.x);
            if (i < row_width)
                *reinterpret_cast<float4*>(raw + i) = make_float4(v[u].x * w[u].x, v[u].y * w[u].y, v[u].z * w[u].z, v[u].w * w[u].w);
            const float ss = v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
            if (i < q_width) ssq += ss;
            else if (i < qk_width) ssk += ss;
        }
    }
    const int table_row = pos < p.table_positions ? pos : p.table_positions - 1;   // positions are checked on the host
    if (!p.tables_final)
        for (int j = threadIdx.x; j < half; j += NORM_BLOCK) {
            s_cos[j] = p.cos_table[(size_t)table_row * half + j];
            s_sin[j] = p.sin_table[(size_t)table_row * half + j];
        }
    const int page = p.tables_final ? page_early : p.write_cache ? p.page_table[(size_t)slot * p.max_pages + pos / FRB_PAGE] : -1;
    const int in_page = pos % FRB_PAGE;
    float rinv_q = 1.f, rinv_k = 1.f;
    if (qw || kw) {
        block_sum_pair<NORM_BLOCK>(ssq, ssk, scratch);
        if (qw) rinv_q = 1.0f / sqrtf(ssq / (float)q_width + p.eps);
        if (kw) rinv_k = 1.0f / sqrtf(ssk / (float)k_width + p.eps);
    } else {
        __syncthreads();
    }

    for (int i = 4 * threadIdx.x; i < qk_width; i += 4 * NORM_BLOCK) {
        const bool is_q = i < q_width;
        const float* base = is_q ? raw : raw + q_width;
        const float rinv = is_q ? rinv_q : rinv_k;
        const int local = is_q ? i : i - q_width;
        const int head = (int)__umulhi((unsigned)local, p.head_dim_inverse), dim = local - head * hd;   // local / hd
        float4 a = *reinterpret_cast<const float4*>(base + local);
        a = make_float4(a.x * rinv, a.y * rinv, a.z * rinv, a.w * rinv);
        if (dim < p.rotary_dim) {
            // a' = a c - b s ; b' = b c + a s   (src/minimax.rs:78-81)
            if (p.interleaved) {                 // pairs (x, y) and (z, w) of this group, angles dim/2 and dim/2 + 1
                const int j = dim >> 1;
                const float c0 = s_cos[j], s0 = s_sin[j], c1 = s_cos[j + 1], s1 = s_sin[j + 1];
                a = make_float4(a.x * c0 - a.y * s0, a.y * c0 + a.x * s0, a.z * c1 - a.w * s1, a.w * c1 + a.z * s1);
            } else {
                const bool first = dim < half;
                const int j = first ? dim : dim - half;
                float4 b = *reinterpret_cast<const float4*>(base + (first ? local + half : local - half));
                b = make_float4(b.x * rinv, b.y * rinv, b.z * rinv, b.w * rinv);
                const float4 c = *reinterpret_cast<const float4*>(s_cos + j), sn = *reinterpret_cast<const float4*>(s_sin + j);
                if (first) a = make_float4(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w);
                else a = make_float4(a.x * c.x + b.x * sn.x, a.y * c.y + b.y * sn.y, a.z * c.z + b.z * sn.z, a.w * c.w + b.w * sn.w);
            }
        }
        if (is_q) {
            store4<OutT>((OutT*)p.q_out + (size_t)t * q_width + local, a);
        } else if (page >= 0) {
            const size_t at = (((size_t)page * p.num_kv_heads + head) * FRB_PAGE + in_page) * hd + dim;
            store4<OutT>((OutT*)p.k_pages + at, a);
        }
    }
    if (page >= 0 && !p.v_tiles) {
        const float* vrow = raw + qk_width;
        for (int i = threadIdx.x; i < k_width; i += NORM_BLOCK) {
            const int head = (int)__umulhi((unsigned)i, p.head_dim_inverse), dim = i - head * hd;
            const size_t at = (((size_t)page * p.num_kv_heads + head) * hd + dim) * FRB_PAGE + in_page;
            ((OutT*)p.v_pages)[at] = from_f32<OutT>(vrow[i]);
        }
    }
}

FRB_API int frb_qkv_prepare(const void* qkv, int in_dtype, const void* q_weight, const void* k_weight, int weight_dtype,
                            float eps, const float* cos_table, const float* sin_table, int table_positions,
                            const int* tok_pos, const int* tok_slot, const int* page_table, int max_pages,
                            void* q_out, void* k_pages, void* v_pages, int out_dtype, int num_tokens, int num_heads,
                            int num_kv_heads, int head_dim, int rotary_dim, int interleaved, int write_cache,
                            int per_head, int tables_final, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(rotary_dim % 2 == 0 && rotary_dim <= head_dim, "qkv_prepare: rotary_dim %d must be even and <= head_dim %d",
                  rotary_dim, head_dim);
    FRB_CHECK_ARG(rotary_dim == 0 || (cos_table && sin_table && table_positions > 0), "qkv_prepare: rotary tables are missing");
    QkvParams p;
    p.qkv = qkv; p.q_weight = q_weight; p.k_weight = k_weight; p.cos_table = cos_table; p.sin_table = sin_table;
    p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.page_table = page_table; p.q_out = q_out; p.k_pages = k_pages;
    p.v_pages = v_pages; p.eps = eps; p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
    p.rotary_dim = rotary_dim; p.interleaved = interleaved; p.max_pages = max_pages; p.write_cache = write_cache;
    p.table_positions = table_positions;
    p.num_tokens = num_tokens; p.v_tiles = 0; p.per_head = per_head && (q_weight || k_weight);
    p.tables_final = tables_final;
    p.head_dim_inverse = (unsigned)((0x100000000ull + (unsigned)head_dim - 1) / (unsigned)head_dim);
    FRB_CHECK_ARG((long long)(num_heads + 2 * num_kv_heads) * head_dim < (1 << 24), "qkv_prepare: %d heads of %d", num_heads, head_dim);
    // per-head statistics: the squares of the q and k rows and one factor per head beside the rows
    const size_t smem = ((size_t)(num_heads + 2 * num_kv_heads) * head_dim + rotary_dim +
                         (p.per_head ? (size_t)(num_heads + num_kv_heads) * (head_dim + 1) : 0)) * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "qkv_prepare: (heads + 2 kv heads) * head_dim = %d needs more than 200 KB of shared memory",
                  (num_heads + 2 * num_kv_heads) * head_dim);
    const int in_bytes = in_dtype == FRB_F32 ? 4 : 2, out_bytes = out_dtype == FRB_F32 ? 4 : 2, w_bytes = weight_dtype == FRB_F32 ? 4 : 2;
    const auto aligned = [](const void* ptr, int bytes) { return ((uintptr_t)ptr & (size_t)(4 * bytes - 1)) == 0; };
    const bool by_four = !p.per_head && head_dim % 4 == 0 && rotary_dim % (interleaved ? 4 : 8) == 0 && aligned(qkv, in_bytes) &&
                         aligned(q_out, out_bytes) && aligned(k_pages, out_bytes) && aligned(q_weight, w_bytes) &&
                         aligned(k_weight, w_bytes);
    FRB_DISPATCH_DTYPE(in_dtype, InT, FRB_DISPATCH_DTYPE(out_dtype, OutT, FRB_DISPATCH_DTYPE(weight_dtype, WT, {
        if (num_tokens <= NORM_FEW_ROWS) {
            auto kernel = by_four ? qkv_prepare_vec_kernel<InT, OutT, WT, 1024> : qkv_prepare_kernel<InT, OutT, WT, 1024>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_tokens), dim3(1024), smem, stream, p);
        } else if (by_four && write_cache) {
            // many tokens: the values go through blocks of their own (64 tokens of a kv head), which write them
            // along the tokens instead of one two-byte store per token and dimension

            const size_t tile_bytes = (size_t)head_dim * (QKV_V_TOKENS + 2) * sizeof(OutT);
            const size_t bytes = smem > tile_bytes ? smem : tile_bytes;
            auto kernel = qkv_prepare_vec_kernel<InT, OutT, WT, 256>;
            if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            const int v_blocks = (num_tokens + QKV_V_TOKENS - 1) / QKV_V_TOKENS * num_kv_heads;
            p.v_tiles = v_blocks;
            launch_dependent(kernel, dim3(num_tokens + v_blocks), dim3(256), bytes, stream, p);
        } else {
            auto kernel = by_four ? qkv_prepare_vec_kernel<InT, OutT, WT, 256> : qkv_prepare_kernel<InT, OutT, WT, 256>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_tokens), dim3(256), smem, stream, p);
        }
    })));
    FRB_RETURN_LAUNCH("qkv_prepare");
}

// ----------------------------------------------------------------------------- small helpers

// x[i] += delta[i]  (float32 residual sum when no norm follows)
__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ delta, size_t n) {
    after_previous_kernel();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += delta[i];
}

FRB_API int frb_add_rows(float* x, const float* delta, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    launch_dependent(add_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, delta, (size_t)n);
    FRB_RETURN_LAUNCH("add_rows");
}

// out[t, i] = silu(both[t, i]) * both[t, width + i], silu(x) = x / (1 + exp(-x))  (src/minimax.rs:31,119)
template <typename OutT>
__global__ void gated_unit_kernel(const float* __restrict__ both, OutT* __restrict__ out, int width, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / width, c = i - t * width;
    const float g = both[t * 2 * width + c], u = both[t * 2 * width + width + c];
    out[i] = from_f32<OutT>(g / (1.0f + expf(-g)) * u);
}

FRB_API int frb_gated_unit(const float* both, void* out, int out_dtype, int rows, int width, cudaStream_t stream) {
    const size_t total = (size_t)rows * width;
    if (total == 0) return 0;
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        gated_unit_kernel<OutT><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(both, (OutT*)out, width, total);
    });
    FRB_RETURN_LAUNCH("gated_unit");
}
