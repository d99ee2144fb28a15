// One-token attention over the cache with the pages brought into shared memory by TMA (bfloat16, head
// sizes 64 and 128).
//
// The formula is the reference's (src/minimax.rs:270-281) and the arithmetic is that of
// attention_decode_mma_kernel: a block takes 256 keys (four pages) of one kv head of one sequence, each of
// four warps one page: scores with mma.sync, softmax within the page, P V, and the four results combined
// through shared memory; the merge kernel then adds the chunks in order.  What differs is how the keys and
// values arrive.  There each warp loads its operands from global memory into registers, a few at a time, and
// a step with a long context is bound by the latency of those loads.  Here a fifth warp asks for all of the
// block's pages at once: every page's keys [64][HD] and transposed values [HD][64] are copied by
// cp.async.bulk.tensor into a stage of shared memory (128-byte swizzle) and announced on an mbarrier, so that
// two blocks per SM keep close to 200 KB in flight.  Six stages hold the four pages' keys and the first two
// pages' values; the values of pages 2 and 3 follow into the stages of the keys of pages 0 and 1 once those
// have been multiplied.
//
// Which key a lane's column of the score tile stands for, and which dimension its column of the output tile,
// is free (softmax and the sum over keys do not care): they are chosen so that the eight lanes of a quarter
// warp read rows that differ in bit 2, which under the swizzle are the two halves of the banks.
//
// Every wait on an mbarrier gives up after about a second and sets `status`; the block then skips its work,
// waits (with the same limit) for the copies it has asked for, and returns.
#include "attention_mma.cuh"
#include "tma.cuh"

#define DT_STAGES 6
#define DT_THREADS 160         // warps 0-3: one page each; warp 4: asks for the copies
#define DT_PAGES (ATT_CHUNK / FRB_PAGE)

using namespace frb_tma;

template <int HD>
__global__ void __launch_bounds__(DT_THREADS, 2)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            DecodeAttnParams p, int* status) {
    after_previous_kernel();
    static_assert(DT_PAGES == 4, "four warps take the four pages of a chunk");
    constexpr int STAGE_BYTES = FRB_PAGE * HD * 2;
    constexpr int O_STRIDE = HD + 8;
    static_assert(16 * O_STRIDE * 4 <= STAGE_BYTES, "a warp's partial result fits into a stage");
    extern __shared__ uint8_t dynamic[];
    __shared__ uint64_t full_k[DT_PAGES], full_v[DT_PAGES], free_k[2];
    __shared__ float sm_m[4][16], sm_l[4][16];
    __shared__ int failed;
    uint8_t* stages = reinterpret_cast<uint8_t*>(((uintptr_t)dynamic + 1023) & ~(uintptr_t)1023);

    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int group = p.num_heads / p.num_kv_heads;
    const int pos = p.seq_pos[b];
    const int slot = p.seq_slot[b];               // asked for together with the position: one wait, not two
    const int hi_key = pos, lo_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    if (chunk * ATT_CHUNK > hi_key || (chunk + 1) * ATT_CHUNK <= lo_key) return;      // the merge skips these chunks

    const int first_page = chunk * DT_PAGES;
    const auto holds_keys = [&](int w) {          // whether page w of the chunk has a key that the token may see
        const int key_base = (first_page + w) * FRB_PAGE;
        return key_base <= hi_key && key_base + FRB_PAGE > lo_key;
    };
    // keys of page w: stage w; values of page w: stage 4 + w for the first two pages, stage w - 2 for the others
    const auto stage_k = [&](int w) { return stages + (size_t)w * STAGE_BYTES; };
    const auto stage_v = [&](int w) { return stages + (size_t)(w < 2 ? 4 + w : w - 2) * STAGE_BYTES; };

    int page_row[DT_PAGES];                       // the page's first row in [pages * kv heads] rows of pages
    if (threadIdx.x == 0) {
        for (int i = 0; i < DT_PAGES; ++i) { bar_init(&full_k[i], 1); bar_init(&full_v[i], 1); }
        bar_init(&free_k[0], 1);
        bar_init(&free_k[1], 1);
        failed = 0;
        bar_init_fence();
    } else if (threadIdx.x == DT_PAGES * 32) {    // the page numbers are on their way while the barriers are set up
        const int* table = p.page_table + (size_t)slot * p.max_pages + first_page;
        for (int w = 0; w < DT_PAGES; ++w) page_row[w] = holds_keys(w) ? table[w] * p.num_kv_heads + kvh : -1;
    }
    __syncthreads();

    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
    if (warp == DT_PAGES) {
        if (lane == 0) {
            for (int w = 0; w < DT_PAGES; ++w) {
                if (page_row[w] < 0) continue;
                bar_expect(&full_k[w], STAGE_BYTES);
                for (int x = 0; x < HD / 64; ++x)
                    load_2d(stage_k(w) + (size_t)x * FRB_PAGE * 128, &map_k, 64 * x, page_row[w] * FRB_PAGE, &full_k[w]);
            }
            for (int w = 0; w < DT_PAGES; ++w) {
                if (page_row[w] < 0) continue;
                if (w >= 2 && !bar_wait(&free_k[w - 2], 0, &failed)) break;
                bar_expect(&full_v[w], STAGE_BYTES);
                load_2d(stage_v(w), &map_v, 0, page_row[w] * HD, &full_v[w]);
            }
        }
    } else if (holds_keys(warp)) {
        const int key_base = (first_page + warp) * FRB_PAGE;
        const bf16* q_base = p.q + ((size_t)b * p.num_heads + (size_t)kvh * group) * HD;
        const bf16* q0 = g < group ? q_base + (size_t)g * HD : nullptr;
        const bf16* q1 = g + 8 < group ? q_base + (size_t)(g + 8) * HD : nullptr;
        uint4 q[HD / 32][2];
#pragma unroll
        for (int step = 0; step < HD / 32; ++step) {
            q[step][0] = q0 ? __ldg(reinterpret_cast<const uint4*>(q0 + 32 * step) + t) : make_uint4(0, 0, 0, 0);
            q[step][1] = q1 ? __ldg(reinterpret_cast<const uint4*>(q1 + 32 * step) + t) : make_uint4(0, 0, 0, 0);
        }
        float s[8][4];
        bool ok = bar_wait(&full_k[warp], 0, &failed);
        if (ok) {
            const uint8_t* keys = stage_k(warp);
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    // column g of this score tile is key 32 m + 8 (g >> 1) + 4 (g & 1) + u of the page
                    const int key_local = 32 * m + 8 * (g >> 1) + 4 * (g & 1) + u;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int step = 0; step < HD / 32; ++step) {
                        const int c = 4 * (step & 1) + t;           // 16-byte chunk within the row's 128 bytes
                        const uint4 kb = *reinterpret_cast<const uint4*>(keys + (size_t)(step >> 1) * FRB_PAGE * 128 +
                                                                         key_local * 128 + ((c ^ (key_local & 7)) << 4));
                        mma_bf16(acc, q[step][0].x, q[step][1].x, q[step][0].y, q[step][1].y, kb.x, kb.y);
                        mma_bf16(acc, q[step][0].z, q[step][1].z, q[step][0].w, q[step][1].w, kb.z, kb.w);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key_base + 32 * m + 8 * t + 4 * (e & 1) + u;     // column 2 t + (e & 1)
                        const float v = (key >= lo_key && key <= hi_key) ? acc[e] * p.scale2 : -INFINITY;
                        s[4 * m + u][e] = v;
                        row_max[e >> 1] = fmaxf(row_max[e >> 1], v);
                    }
                }
        }
        __syncwarp();
        if (warp < 2 && lane == 0) bar_arrive(&free_k[warp]);          // this page's keys are no longer needed
        if (ok) {
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
            // the thread's weights of keys 32 m + 8 t .. + 7 in the order of memory: key 4 e + u sits in s[4 m + u][e]
            uint32_t pa[2][4], pb[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                pa[m][0] = pack_bf16(s[4 * m][0], s[4 * m + 1][0]);     pa[m][1] = pack_bf16(s[4 * m][2], s[4 * m + 1][2]);
                pa[m][2] = pack_bf16(s[4 * m + 2][0], s[4 * m + 3][0]); pa[m][3] = pack_bf16(s[4 * m + 2][2], s[4 * m + 3][2]);
                pb[m][0] = pack_bf16(s[4 * m][1], s[4 * m + 1][1]);     pb[m][1] = pack_bf16(s[4 * m][3], s[4 * m + 1][3]);
                pb[m][2] = pack_bf16(s[4 * m + 2][1], s[4 * m + 3][1]); pb[m][3] = pack_bf16(s[4 * m + 2][3], s[4 * m + 3][3]);
            }
            ok = bar_wait(&full_v[warp], 0, &failed);
            if (ok) {
                const uint8_t* values = stage_v(warp);
                float o[HD / 8][4];
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
                    // column g of this output tile is dimension 8 n + 4 (g & 1) + (g >> 1)
                    const int dim = 8 * n + 4 * (g & 1) + (g >> 1);
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        const int c = 4 * m + t;                    // keys 32 m + 8 t .. + 7 of the transposed row
                        const uint4 vb = *reinterpret_cast<const uint4*>(values + dim * 128 + ((c ^ (dim & 7)) << 4));
                        mma_bf16(o[n], pa[m][0], pa[m][1], pa[m][2], pa[m][3], vb.x, vb.y);
                        mma_bf16(o[n], pb[m][0], pb[m][1], pb[m][2], pb[m][3], vb.z, vb.w);
                    }
                }
                __syncwarp();                                       // every lane has read the values: the stage is free
                float* mine = reinterpret_cast<float*>(stage_v(warp));
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) {                  // column 2 t + e is dimension 8 n + 4 e + t
                    mine[g * O_STRIDE + 8 * n + t] = o[n][0];
                    mine[g * O_STRIDE + 8 * n + 4 + t] = o[n][1];
                    mine[(g + 8) * O_STRIDE + 8 * n + t] = o[n][2];
                    mine[(g + 8) * O_STRIDE + 8 * n + 4 + t] = o[n][3];
                }
            }
        }
        if (!ok) row_sum[0] = row_sum[1] = 0.f;
    } else if (warp < 2 && lane == 0) {
        bar_arrive(&free_k[warp]);
    }
    if (warp < DT_PAGES && t == 0) {
        sm_m[warp][g] = row_max[0]; sm_l[warp][g] = row_sum[0];
        sm_m[warp][g + 8] = row_max[1]; sm_l[warp][g + 8] = row_sum[1];
    }
    __syncthreads();
    if (failed) {
        // leave only when the copies that were asked for have landed (or a second limit has passed)
        if (threadIdx.x == 0) {
            *status = 4;
            int again = 0;
            for (int w = 0; w < DT_PAGES; ++w)
                if (holds_keys(w)) { again = 0; bar_wait(&full_k[w], 0, &again); again = 0; bar_wait(&full_v[w], 0, &again); }
        }
        __syncthreads();
        return;
    }
    for (int idx = threadIdx.x; idx < group * HD; idx += DT_THREADS) {
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
                acc += reinterpret_cast<const float*>(stage_v(w))[r * O_STRIDE + d] * f;
            }
        }
        const size_t row = ((size_t)b * p.num_heads + (size_t)kvh * group + r) * p.max_chunks + chunk;
        p.part_o[row * HD + d] = acc;
        if (d == 0) { p.part_ml[row * 2] = top; p.part_ml[row * 2 + 1] = sum; }
    }
}

// As frb_attention_decode_mma, for head sizes 64 and 128.  num_pages: pages of the cache group (the tensor
// maps cover all of them).  status: one int on the device, zero before the call; 4 afterwards if a wait gave up.
FRB_API int frb_attention_decode_tma(const void* q, const void* k_pages, const void* v_pages, int num_pages,
                                     const int* page_table, int max_pages, const int* seq_pos, const int* seq_slot,
                                     float* part_o, float* part_ml, void* out, int num_seqs, int num_heads, int num_kv_heads,
                                     int head_dim, float scale, int window, int max_chunks, int* status, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    const int group = num_kv_heads > 0 ? num_heads / num_kv_heads : 0;
    FRB_CHECK_ARG(num_kv_heads > 0 && num_heads % num_kv_heads == 0 && group <= 16,
                  "attention_decode_tma: %d heads over %d kv heads (groups of at most 16)", num_heads, num_kv_heads);
    FRB_CHECK_ARG(head_dim == 64 || head_dim == 128, "attention_decode_tma: head_dim %d is neither 64 nor 128", head_dim);
    FRB_CHECK_ARG(num_seqs <= 65535 && num_kv_heads <= 65535, "attention_decode_tma: %d sequences exceed the grid", num_seqs);
    CUtensorMap map_k, map_v;
    const uint64_t kv_rows = (uint64_t)num_pages * num_kv_heads;
    FRB_CHECK_ARG(map_rows_of_64(&map_k, k_pages, kv_rows * FRB_PAGE, head_dim, FRB_PAGE) &&
                  map_rows_of_64(&map_v, v_pages, kv_rows * head_dim, FRB_PAGE, head_dim),
                  "attention_decode_tma: cuTensorMapEncodeTiled failed or is not available");
    DecodeAttnParams p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages; p.page_table = page_table;
    p.seq_pos = seq_pos; p.seq_slot = seq_slot; p.part_o = part_o; p.part_ml = part_ml; p.out = (bf16*)out;
    p.scale2 = scale * 1.4426950408889634f; p.window = window; p.max_pages = max_pages; p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads; p.max_chunks = max_chunks;
    dim3 grid(max_chunks, num_kv_heads, num_seqs), merge_grid(num_heads, num_seqs);
    const size_t smem = (size_t)DT_STAGES * FRB_PAGE * head_dim * 2 + 1024;
    if (head_dim == 64) {
        cudaFuncSetAttribute(attention_decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(attention_decode_tma_kernel<64>, grid, dim3(DT_THREADS), smem, stream, map_k, map_v, p, status);
        launch_dependent(attention_decode_merge_kernel<64>, merge_grid, dim3(64), 0, stream, p);
    } else {
        cudaFuncSetAttribute(attention_decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(attention_decode_tma_kernel<128>, grid, dim3(DT_THREADS), smem, stream, map_k, map_v, p, status);
        launch_dependent(attention_decode_merge_kernel<128>, merge_grid, dim3(128), 0, stream, p);
    }
    FRB_RETURN_LAUNCH("attention_decode_tma");
}
