// One-token attention over the cache with the pages brought into shared memory by TMA (bfloat16, head
// sizes 64 and 128).
//
// The formula is the reference's (src/minimax.rs:270-281).  A block takes a run of pages of one kv head of
// one sequence: `chunks_per_block` chunks of 256 keys.  Three warps take the run's pages in turn (warp w the
// pages w, w + 3, ...): scores with mma.sync, a running softmax over the warp's own pages (maximum, sum and
// output rescaled when the maximum grows), P V into the warp's accumulators; at the end the three warps'
// results are combined through shared memory and written as one partial result, and the merge kernel adds
// the blocks' partial results in order.
//
// A fourth warp asks for the pages: every page's keys [64][HD] and transposed values [HD][64] are copied by
// cp.async.bulk.tensor into shared memory (128-byte swizzle).  Each warp has a stage for keys and a stage for
// values of its own, each announced on an mbarrier and given back on another once the warp has multiplied
// it; the next page's keys are on their way while the warp is at the present page's softmax and values.
// The copies run through the whole run of pages, so that a block always has up to 96 KB on the way (two
// blocks per SM), where loads into registers wait for one another and a block of four pages spends a quarter
// of its life on set-up and on combining.  A stage belongs to one warp because a wait on an mbarrier names
// only the parity of the phase it waits for: a warp that used a stage two phases ago cannot tell the phase
// before its own from its own.
//
// Which key a lane's column of the score tile stands for, and which dimension its column of the output tile,
// is free (softmax and the sum over keys do not care): they are chosen so that the eight lanes of a quarter
// warp read rows that differ in bit 2, which under the swizzle are the two halves of the banks.
//
// Every wait on an mbarrier gives up after about a second and sets `status`; the block then skips its work,
// waits (with the same limit) for the copies it has asked for, and returns.
#include "attention_mma.cuh"
#include "tma.cuh"

#define DT_WARPS 3             // warps that multiply
#define DT_STAGES (2 * DT_WARPS)
#define DT_THREADS (32 * (DT_WARPS + 1))   // warps 0-2: the pages in turn; warp 3: asks for the copies
#define DT_CHUNK_PAGES (ATT_CHUNK / FRB_PAGE)
#define DT_RAISE 8.0f          // the running maximum follows a page's maximum only beyond this margin

using namespace frb_tma;

struct DecodeTmaParams {
    DecodeAttnParams a;        // max_chunks: partial results per (sequence, head) = blocks along a sequence
    int chunks_per_block;
    int early;                 // copies go out before the kernel before this one has ended (0: FIELDRUN_B200_ATTENTION_EARLY=0)
    int* status;
};

// Warp w's page number n (the run's page 3 n + w) has its keys in stage 2 w and its values in stage 2 w + 1,
// each on that stage's use n.
template <int HD>
__global__ void __launch_bounds__(DT_THREADS, 2)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            DecodeTmaParams params) {
    // The keys and values of earlier tokens, the page table and the positions do not depend on the kernel before this
    // one (it writes the queries and the new token's key and value): the copies of every page but the sequence's last
    // go out before that kernel has ended; the warps that multiply wait for it before they read the queries.
    let_next_kernel_start();
    const DecodeAttnParams& p = params.a;
    constexpr int STAGE_BYTES = FRB_PAGE * HD * 2;
    constexpr int O_STRIDE = HD + 8;
    static_assert(16 * O_STRIDE * 4 <= STAGE_BYTES, "a warp's partial result fits into a stage");
    extern __shared__ uint8_t dynamic[];
    __shared__ uint64_t full[DT_STAGES], empty[DT_STAGES];
    __shared__ float sm_m[DT_WARPS][16], sm_l[DT_WARPS][16];
    __shared__ int failed;
    uint8_t* stages = reinterpret_cast<uint8_t*>(((uintptr_t)dynamic + 1023) & ~(uintptr_t)1023);

    const int part = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int group = p.num_heads / p.num_kv_heads;
    const int pos = p.seq_pos[b];
    const int slot = p.seq_slot[b];               // asked for together with the position: one wait, not two
    const int hi_key = pos, lo_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    // the pages of this block that hold a key the token may see
    const int pages_per_block = params.chunks_per_block * DT_CHUNK_PAGES;
    const int first_page = max(part * pages_per_block, lo_key / FRB_PAGE);
    const int end_page = min((part + 1) * pages_per_block, hi_key / FRB_PAGE + 1);
    const int num_pages = end_page - first_page;
    if (num_pages <= 0) return;                   // the merge skips these blocks

    if (threadIdx.x == 0) {
        for (int s = 0; s < DT_STAGES; ++s) { bar_init(&full[s], 1); bar_init(&empty[s], 1); }
        failed = 0;
        bar_init_fence();
    }
    __syncthreads();

    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    bool ok = true;

    if (warp == DT_WARPS) {
        if (lane == 0) {
            const int* table = p.page_table + (size_t)slot * p.max_pages + first_page;
            const int rounds = (num_pages + DT_WARPS - 1) / DT_WARPS;
            const int newest = hi_key / FRB_PAGE - first_page;            // the page that the kernel before this one writes to
            bool waited = false;
            if (!params.early) { wait_for_previous_kernel(); waited = true; }
            for (int n = 0; n < rounds && ok; ++n) {
                if (!waited && DT_WARPS * n + DT_WARPS > newest) { wait_for_previous_kernel(); waited = true; }
                int rows[DT_WARPS];               // each page's first row in [pages * kv heads] rows of pages
#pragma unroll
                for (int w = 0; w < DT_WARPS; ++w)
                    rows[w] = DT_WARPS * n + w < num_pages ? table[DT_WARPS * n + w] * p.num_kv_heads + kvh : -1;
#pragma unroll
                for (int half = 0; half < 2; ++half) {                 // the round's keys, then its values
#pragma unroll
                    for (int w = 0; w < DT_WARPS; ++w) {
                        if (rows[w] < 0 || !ok) continue;
                        const int s = 2 * w + half;
                        if (n >= 1 && !bar_wait(&empty[s], (uint32_t)((n - 1) & 1), &failed)) { ok = false; continue; }
                        uint8_t* dst = stages + (size_t)s * STAGE_BYTES;
                        bar_expect(&full[s], STAGE_BYTES);
                        if (half == 0) {
#pragma unroll
                            for (int x = 0; x < HD / 64; ++x)
                                load_2d(dst + (size_t)x * FRB_PAGE * 128, &map_k, 64 * x, rows[w] * FRB_PAGE, &full[s]);
                        } else {
                            load_2d(dst, &map_v, 0, rows[w] * HD, &full[s]);
                        }
                    }
                }
            }
        }
    } else {
        wait_for_previous_kernel();
        const bf16* q_base = p.q + ((size_t)b * p.num_heads + (size_t)kvh * group) * HD;
        const bf16* q0 = g < group ? q_base + (size_t)g * HD : nullptr;
        const bf16* q1 = g + 8 < group ? q_base + (size_t)(g + 8) * HD : nullptr;
        uint4 q[HD / 32][2];
#pragma unroll
        for (int step = 0; step < HD / 32; ++step) {
            q[step][0] = q0 ? __ldg(reinterpret_cast<const uint4*>(q0 + 32 * step) + t) : make_uint4(0, 0, 0, 0);
            q[step][1] = q1 ? __ldg(reinterpret_cast<const uint4*>(q1 + 32 * step) + t) : make_uint4(0, 0, 0, 0);
        }
        for (int n = 0; DT_WARPS * n + warp < num_pages && ok; ++n) {
            const int key_base = (first_page + DT_WARPS * n + warp) * FRB_PAGE;
            const int k_stage = 2 * warp, v_stage = 2 * warp + 1;
            const uint32_t parity = (uint32_t)(n & 1);
            float s[8][4];
            ok = bar_wait(&full[k_stage], parity, &failed);
            if (!ok) break;
            {
                const uint8_t* keys = stages + (size_t)k_stage * STAGE_BYTES;
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        // column g of this score tile is key 32 m + 8 (g >> 1) + 4 (g & 1) + u of the page
                        const int key_local = 32 * m + 8 * (g >> 1) + 4 * (g & 1) + u;
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int step = 0; step < HD / 32; ++step) {
                            const int c = 4 * (step & 1) + t;       // 16-byte chunk within the row's 128 bytes
                            const uint4 kb = *reinterpret_cast<const uint4*>(keys + (size_t)(step >> 1) * FRB_PAGE * 128 +
                                                                             key_local * 128 + ((c ^ (key_local & 7)) << 4));
                            mma_bf16(acc, q[step][0].x, q[step][1].x, q[step][0].y, q[step][1].y, kb.x, kb.y);
                            mma_bf16(acc, q[step][0].z, q[step][1].z, q[step][0].w, q[step][1].w, kb.z, kb.w);
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) s[4 * m + u][e] = acc[e] * p.scale2;
                    }
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&empty[k_stage]);                  // this page's keys are no longer needed
            // only a run's first and last page can hold keys the token may not see
            if (key_base < lo_key || key_base + FRB_PAGE - 1 > hi_key) {
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int key = key_base + 32 * m + 8 * t + 4 * (e & 1) + u;     // column 2 t + (e & 1)
                            if (key < lo_key || key > hi_key) s[4 * m + u][e] = -INFINITY;
                        }
            }
            float page_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) page_max[e >> 1] = fmaxf(page_max[e >> 1], s[j][e]);
            float corr[2];
            bool grew = false;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                page_max[r] = fmaxf(page_max[r], __shfl_xor_sync(0xffffffffu, page_max[r], 1));
                page_max[r] = fmaxf(page_max[r], __shfl_xor_sync(0xffffffffu, page_max[r], 2));
                // the page holds at least one visible key, and every row sees the same keys: the maxima are finite
                corr[r] = 1.f;
                if (page_max[r] > row_max[r] + DT_RAISE) {           // also on the warp's first page
                    corr[r] = exp2f(row_max[r] - page_max[r]);
                    row_max[r] = page_max[r];
                    grew = true;
                }
            }
            if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
                for (int n2 = 0; n2 < HD / 8; ++n2) {
                    o[n2][0] *= corr[0]; o[n2][1] *= corr[0];
                    o[n2][2] *= corr[1]; o[n2][3] *= corr[1];
                }
            }
            float page_sum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[j][e] - row_max[e >> 1]);
                    s[j][e] = pv;
                    page_sum[e >> 1] += pv;
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                page_sum[r] += __shfl_xor_sync(0xffffffffu, page_sum[r], 1);
                page_sum[r] += __shfl_xor_sync(0xffffffffu, page_sum[r], 2);
                row_sum[r] = row_sum[r] * corr[r] + page_sum[r];
            }
            // the thread's weights of keys 32 m + 8 t .. + 7 in the order of memory: key 4 e + u sits in s[4 m + u][e]
            uint32_t pa[2][4], pb[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                pa[m][0] = pack_bf16(s[4 * m][0], s[4 * m + 1][0]);     pa[m][1] = pack_bf16(s[4 * m][2], s[4 * m + 1][2]);
                pa[m][2] = pack_bf16(s[4 * m + 2][0], s[4 * m + 3][0]); pa[m][3] = pack_bf16(s[4 * m + 2][2], s[4 * m + 3][2]);
                pb[m][0] = pack_bf16(s[4 * m][1], s[4 * m + 1][1]);     pb[m][1] = pack_bf16(s[4 * m][3], s[4 * m + 1][3]);
                pb[m][2] = pack_bf16(s[4 * m + 2][1], s[4 * m + 3][1]); pb[m][3] = pack_bf16(s[4 * m + 2][3], s[4 * m + 3][3]);
            }
            ok = bar_wait(&full[v_stage], parity, &failed);
            if (!ok) break;
            {
                const uint8_t* values = stages + (size_t)v_stage * STAGE_BYTES;
#pragma unroll
                for (int n2 = 0; n2 < HD / 8; ++n2) {
                    // column g of this output tile is dimension 8 n2 + 4 (g & 1) + (g >> 1)
                    const int dim = 8 * n2 + 4 * (g & 1) + (g >> 1);
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        const int c = 4 * m + t;                    // keys 32 m + 8 t .. + 7 of the transposed row
                        const uint4 vb = *reinterpret_cast<const uint4*>(values + dim * 128 + ((c ^ (dim & 7)) << 4));
                        mma_bf16(o[n2], pa[m][0], pa[m][1], pa[m][2], pa[m][3], vb.x, vb.y);
                        mma_bf16(o[n2], pb[m][0], pb[m][1], pb[m][2], pb[m][3], vb.z, vb.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&empty[v_stage]);                  // nor are its values
        }
        if (!ok) row_sum[0] = row_sum[1] = 0.f;
    }
    __syncthreads();                   // every copy that was asked for has been waited for: the stages are free
    if (failed) {
        // leave only when the copies that were asked for have landed (or a second limit has passed)
        if (threadIdx.x == 0) {
            *params.status = 4;
            for (int s = 0; s < DT_STAGES; ++s) { int again = 0; bar_wait(&full[s], 0, &again); }
        }
        __syncthreads();
        return;
    }
    if (warp < DT_WARPS) {
        float* mine = reinterpret_cast<float*>(stages + (size_t)warp * STAGE_BYTES);
#pragma unroll
        for (int n2 = 0; n2 < HD / 8; ++n2) {                       // column 2 t + e is dimension 8 n2 + 4 e + t
            mine[g * O_STRIDE + 8 * n2 + t] = o[n2][0];
            mine[g * O_STRIDE + 8 * n2 + 4 + t] = o[n2][1];
            mine[(g + 8) * O_STRIDE + 8 * n2 + t] = o[n2][2];
            mine[(g + 8) * O_STRIDE + 8 * n2 + 4 + t] = o[n2][3];
        }
        if (t == 0) {
            sm_m[warp][g] = row_max[0]; sm_l[warp][g] = row_sum[0];
            sm_m[warp][g + 8] = row_max[1]; sm_l[warp][g + 8] = row_sum[1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += DT_THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < DT_WARPS; ++w) top = fmaxf(top, sm_m[w][r]);
        float sum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < DT_WARPS; ++w) {
            if (sm_l[w][r] > 0.f) {                             // a warp that had no page wrote zeros and no maximum
                const float f = exp2f(sm_m[w][r] - top);
                sum += sm_l[w][r] * f;
                acc += reinterpret_cast<const float*>(stages + (size_t)w * STAGE_BYTES)[r * O_STRIDE + d] * f;
            }
        }
        const size_t row = ((size_t)b * p.num_heads + (size_t)kvh * group + r) * p.max_chunks + part;
        p.part_o[row * HD + d] = acc;
        if (d == 0) { p.part_ml[row * 2] = top; p.part_ml[row * 2 + 1] = sum; }
    }
}

// grid (head, sequence): merges the blocks' partial results of one (sequence, head), first block to last.
template <int HD>
__global__ void __launch_bounds__(HD) attention_decode_tma_merge_kernel(DecodeTmaParams params) {
    after_previous_kernel();
    const DecodeAttnParams& p = params.a;
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const int pos = p.seq_pos[b];
    const int lo_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int keys_per_block = params.chunks_per_block * ATT_CHUNK;
    // never beyond the partial results the launch has room for, whatever the position says
    const int last = min(pos / keys_per_block, p.max_chunks - 1), first = min(lo_key / keys_per_block, last);
    if (pos / keys_per_block >= p.max_chunks && d == 0) atomicExch(params.status, FRB_STATUS_TOO_LONG);   // keys were left out
    const size_t row0 = ((size_t)b * p.num_heads + head) * p.max_chunks;
    p.out[((size_t)b * p.num_heads + head) * HD + d] = __float2bfloat16_rn(merged_element<HD>(p.part_ml, p.part_o, row0, first, last, d));
}

// As frb_attention_decode_mma, for head sizes 64 and 128.  num_pages: pages of the cache group (the tensor
// maps cover all of them).  max_chunks: chunks of 256 keys of the longest sequence; part_o and part_ml need
// room for ceil(max_chunks / chunks_per_block) partial results per (sequence, head).  chunks_per_block: chunks
// that one block takes (at least 1).  status: one int on the device, zero before the call; 4 afterwards if a
// wait gave up.
FRB_API int frb_attention_decode_tma(const void* q, const void* k_pages, const void* v_pages, int num_pages,
                                     const int* page_table, int max_pages, const int* seq_pos, const int* seq_slot,
                                     float* part_o, float* part_ml, void* out, int num_seqs, int num_heads, int num_kv_heads,
                                     int head_dim, float scale, int window, int max_chunks, int chunks_per_block, int* status,
                                     cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    const int group = num_kv_heads > 0 ? num_heads / num_kv_heads : 0;
    FRB_CHECK_ARG(num_kv_heads > 0 && num_heads % num_kv_heads == 0 && group <= 16,
                  "attention_decode_tma: %d heads over %d kv heads (groups of at most 16)", num_heads, num_kv_heads);
    FRB_CHECK_ARG(head_dim == 64 || head_dim == 128, "attention_decode_tma: head_dim %d is neither 64 nor 128", head_dim);
    FRB_CHECK_ARG(num_seqs <= 65535 && num_kv_heads <= 65535, "attention_decode_tma: %d sequences exceed the grid", num_seqs);
    FRB_CHECK_ARG(chunks_per_block >= 1 && max_chunks >= 1, "attention_decode_tma: %d chunks per block", chunks_per_block);
    CUtensorMap map_k, map_v;
    const uint64_t kv_rows = (uint64_t)num_pages * num_kv_heads;
    FRB_CHECK_ARG(map_rows_of_64(&map_k, k_pages, kv_rows * FRB_PAGE, head_dim, FRB_PAGE) &&
                  map_rows_of_64(&map_v, v_pages, kv_rows * head_dim, FRB_PAGE, head_dim),
                  "attention_decode_tma: cuTensorMapEncodeTiled failed or is not available");
    DecodeTmaParams params;
    DecodeAttnParams& p = params.a;
    const int parts = (max_chunks + chunks_per_block - 1) / chunks_per_block;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages; p.page_table = page_table;
    p.seq_pos = seq_pos; p.seq_slot = seq_slot; p.part_o = part_o; p.part_ml = part_ml; p.out = (bf16*)out;
    p.scale2 = scale * 1.4426950408889634f; p.window = window; p.max_pages = max_pages; p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads; p.max_chunks = parts; p.status = status;
    params.chunks_per_block = chunks_per_block; params.status = status;
    static const int early = [] { const char* v = getenv("FIELDRUN_B200_ATTENTION_EARLY"); return !(v && v[0] == '0'); }();
    params.early = early;
    dim3 grid(parts, num_kv_heads, num_seqs), merge_grid(num_heads, num_seqs);
    const size_t smem = (size_t)DT_STAGES * FRB_PAGE * head_dim * 2 + 1024;
    if (head_dim == 64) {
        cudaFuncSetAttribute(attention_decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent_resident(early ? 2 : 1, attention_decode_tma_kernel<64>, grid, dim3(DT_THREADS), smem, stream, map_k, map_v, params);
        launch_dependent(attention_decode_tma_merge_kernel<64>, merge_grid, dim3(64), 0, stream, params);
    } else {
        cudaFuncSetAttribute(attention_decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent_resident(early ? 2 : 1, attention_decode_tma_kernel<128>, grid, dim3(DT_THREADS), smem, stream, map_k, map_v, params);
        launch_dependent(attention_decode_tma_merge_kernel<128>, merge_grid, dim3(128), 0, stream, params);
    }
    FRB_RETURN_LAUNCH("attention_decode_tma");
}
