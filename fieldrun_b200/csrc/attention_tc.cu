// Many-token attention on the fifth-generation tensor cores (tcgen05), for prompts in bfloat16.
//
// The formula is the reference's (src/minimax.rs:270-281): s = q.k * scale over the keys a query may see,
// p = softmax(s), out = p V.  A block takes 128 queries of one head.  For every step of two cache pages (128 keys):
//   S = Q K^T      tcgen05.mma 128 x 128 x HD, Q and the pages' keys in shared memory (TMA, 128-byte swizzle),
//                  S in tensor memory, two buffers so that the next step's product runs during this step's softmax;
//   softmax        eight warps, two threads per query row, one for each page of the step.  The two keep a running
//                  maximum and sum of their own, as if their pages were two requests' keys: nothing passes between
//                  them until the end.  S comes back with tcgen05.ld; P (bfloat16) goes back into tensor memory
//                  with tcgen05.st, over the columns that the thread's own scores came from;
//   O_h += P_h V_h tcgen05.mma 128 x HD x 64 for page h of the step, with P_h as the tensor-memory operand and the
//                  page's transposed values [HD][64 keys] as the shared-memory operand; each page of a step has an
//                  accumulator of its own (all 512 columns: S/P twice, O twice).
//   the end        out = (O_0 a_0 + O_1 a_1) / (l_0 a_0 + l_1 a_1) with a_h = 2^(m_h - max(m_0, m_1)).
// One warp per scheduler (four in all) could not hide its own latencies: measured with clock stamps, a step's
// softmax then took 1,790 cycles beside 1,600 cycles of MMA issue (8 + 8 MMAs of about 100 cycles each, the
// least that one tcgen05.mma of M 128 takes here whatever N up to 128), and each side waited a quarter of its
// time for the other.
// The running maximum of a row is only raised when the step's maximum exceeds it by more than 8 (in units of
// log2): the weights are then at most 2^8, the result is the same after the division by the row's sum, and
// O has to be rescaled (read, multiplied, written back) only on those rare pages.
//
// Every wait on an mbarrier gives up after about a second (at once when another wait of the block has given
// up), sets `status`, and the block leaves through the common exit, which frees the tensor memory.
#include "tcgen05.cuh"

#define AT_QUERIES 128
#define AT_THREADS 320         // warp 0: TMA producer, warp 1: MMA issuer and tensor-memory owner, warps 2-9: softmax
#define AT_SOFTMAX_THREADS 256 // warps 2-5 take the first page of every step, warps 6-9 the second
#define AT_STAGES 3
#define AT_STEP_PAGES 2        // cache pages per step of the inner loop
#define AT_STEP_KEYS (AT_STEP_PAGES * FRB_PAGE)
#define AT_RAISE 8.0f          // the running maximum follows a page's maximum only beyond this margin

using namespace frb_tma;
using namespace frb_tc;

namespace {

// 2^x by the special-function unit (relative error about 2^-22; -inf and anything below -126 give 0)
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// the largest of three (one instruction on this architecture)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// the hardware's instructions on two float32 values in one 64-bit register
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void halves_of(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pairs(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_pairs(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

}  // namespace

struct AttnTcParams {
    const int* page_table;
    const int* tile_seq;       // [tiles]
    const int* tile_q0;        // [tiles] first row of the tile among its sequence's new tokens
    const int* seq_slot;
    const int* seq_start;
    const int* seq_q_len;
    const int* cu_q_len;
    bf16* out;                 // [T, nh * HD]
    int* status;
    float scale2;              // softmax scale * log2(e)
    int window, max_pages, num_heads, num_kv_heads;
};

// grid (tile of 128 queries, head); the longest tiles of a sequence (its last ones) start first
template <int HD>
__global__ void __launch_bounds__(AT_THREADS)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, AttnTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    // p_full[buffer][page of the step]: that page's probabilities of the buffer's step are in tensor memory
    __shared__ uint64_t q_full, kv_full[AT_STAGES], kv_empty[AT_STAGES], s_full[2], p_full[2][AT_STEP_PAGES];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed_flag;
    volatile int* failed = &failed_flag;
    constexpr int KBLOCKS = HD / 64;                           // 64 dims = one 128-byte swizzled row
    constexpr uint32_t Q_BYTES = AT_QUERIES * HD * 2, K_BYTES = FRB_PAGE * HD * 2, V_BYTES = HD * FRB_PAGE * 2;
    constexpr uint32_t STAGE_BYTES = AT_STEP_PAGES * (K_BYTES + V_BYTES);
    constexpr uint32_t K_BLOCK_BYTES = AT_STEP_KEYS * 128;     // one 64-dim block of a step's keys: [128 keys][128 bytes]
    // Tensor memory: two buffers of 128 columns, each a step's S (a column per key; page h of the step in columns
    // 64 h ...) and then its P (two bfloat16 per column, page h in columns 64 h ... 64 h + 31); O_0 and O_1.
    constexpr uint32_t SP_COL0 = 0, O_COL0 = 2 * AT_STEP_KEYS;
    constexpr uint32_t TMEM_COLS = 512;
    static_assert(O_COL0 + AT_STEP_PAGES * 128 <= TMEM_COLS && HD <= 128 && AT_STEP_PAGES == 2, "tensor memory layout");

    // The step's tables are not the work of the kernel before this one (it writes queries, keys and values): they
    // are read, and barriers and tensor memory set up, while that kernel still runs.
    let_next_kernel_start();
    const int tile = gridDim.x - 1 - blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.num_heads / p.num_kv_heads, kvh = head / group;
    const int b = p.tile_seq[tile], q0 = p.tile_q0[tile];
    const int q_len = p.seq_q_len[b], start = p.seq_start[b], tok0 = p.cu_q_len[b] + q0;
    const int* table = p.page_table + (size_t)p.seq_slot[b] * p.max_pages;
    const int last_key = start + min(q0 + AT_QUERIES - 1, q_len - 1);
    const int first_key = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;
    const int first_page = first_key / FRB_PAGE, num_pages = last_key / FRB_PAGE - first_page + 1;
    const int num_steps = (num_pages + AT_STEP_PAGES - 1) / AT_STEP_PAGES;     // a step: two pages, the last one maybe one

    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = base;                                    // KBLOCKS tiles [128 x 64]
    uint8_t* stage0 = base + Q_BYTES;                          // per stage: K (KBLOCKS tiles [128 keys x 64]) then V^T ([HD x 64] per page)

    if (threadIdx.x == 0) {
        bar_init(&q_full, 1);
        for (int s = 0; s < AT_STAGES; ++s) { bar_init(&kv_full[s], 1); bar_init(&kv_empty[s], 1); }
        for (int i = 0; i < 2; ++i) {
            bar_init(&s_full[i], 1);
            for (int h = 0; h < AT_STEP_PAGES; ++h) bar_init(&p_full[i][h], 4);
        }
        failed_flag = 0;
        bar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_slot, TMEM_COLS);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;
    wait_for_previous_kernel();

    if (warp == 0) {
        if (lane == 0) {
            bar_expect(&q_full, Q_BYTES);
#pragma unroll
            for (int kb = 0; kb < KBLOCKS; ++kb)
                load_2d(q_tile + kb * (AT_QUERIES * 128), &map_q, head * HD + kb * 64, tok0, &q_full);
            for (int j = 0; j < num_steps; ++j) {
                const int s = j % AT_STAGES;
                if (!bar_wait(&kv_empty[s], ((j / AT_STAGES) & 1) ^ 1, failed)) { atomicExch(p.status, 11); break; }
                const int pages = min(AT_STEP_PAGES, num_pages - AT_STEP_PAGES * j);
                uint8_t* dst = stage0 + (size_t)s * STAGE_BYTES;
                bar_expect(&kv_full[s], pages * (K_BYTES + V_BYTES));
                for (int h = 0; h < pages; ++h) {
                    const int page = table[first_page + AT_STEP_PAGES * j + h];
                    const int row = page * p.num_kv_heads + kvh;
#pragma unroll
                    for (int kb = 0; kb < KBLOCKS; ++kb)
                        load_2d(dst + kb * K_BLOCK_BYTES + h * (FRB_PAGE * 128), &map_k, kb * 64, row * FRB_PAGE, &kv_full[s]);
                    load_2d(dst + AT_STEP_PAGES * K_BYTES + h * V_BYTES, &map_v, 0, row * HD, &kv_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // float32 accumulate, bf16 operands, K-major; S: M 128 x N 128 (64 for a step of one page); O_h: M 128 x N HD.
            // The MMAs of this thread run in the order of their issue.  So S of step j + 2 may be asked for into the
            // buffer of step j without a wait: P V of step j, which reads that buffer, was issued before, and was issued
            // only when the softmax of step j had read its S and written its P.
            const uint32_t idesc_o = instr_desc_bf16(AT_QUERIES, HD);
            const uint64_t q_desc = tile_desc(smem_addr(q_tile));
            bool ok = bar_wait(&q_full, 0, failed);
            if (!ok) atomicExch(p.status, 12);
            auto issue_scores = [&](int j) -> bool {
                const int s = j % AT_STAGES;
                if (!bar_wait(&kv_full[s], (j / AT_STAGES) & 1, failed)) { atomicExch(p.status, 13); return false; }
                fence_after_sync();
                const int pages = min(AT_STEP_PAGES, num_pages - AT_STEP_PAGES * j);
                const uint32_t idesc_s = instr_desc_bf16(AT_QUERIES, pages * FRB_PAGE);
                const uint64_t k_desc = tile_desc(smem_addr(stage0 + (size_t)s * STAGE_BYTES));
#pragma unroll
                for (int kb = 0; kb < KBLOCKS; ++kb)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_ss(tmem + SP_COL0 + AT_STEP_KEYS * (j & 1), q_desc + ((kb * (AT_QUERIES * 128) + k * 32) >> 4),
                               k_desc + ((kb * K_BLOCK_BYTES + k * 32) >> 4), idesc_s, (kb | k) != 0);
                mma_commit(&s_full[j & 1]);
                return true;
            };
            if (ok) ok = issue_scores(0);
            bool begun[AT_STEP_PAGES] = {false, false};        // whether O_h holds anything yet
            for (int j = 0; j < num_steps && ok; ++j) {
                if (j + 1 < num_steps) ok = issue_scores(j + 1);
                if (!ok) break;
                const int s = j % AT_STAGES;
                const int pages = min(AT_STEP_PAGES, num_pages - AT_STEP_PAGES * j);
                const uint64_t v_desc = tile_desc(smem_addr(stage0 + (size_t)s * STAGE_BYTES + AT_STEP_PAGES * K_BYTES));
                for (int h = 0; h < pages && ok; ++h) {
                    if (!bar_wait(&p_full[j & 1][h], (j >> 1) & 1, failed)) { atomicExch(p.status, 15); ok = false; break; }
                    fence_after_sync();
#pragma unroll
                    for (int k = 0; k < 4; ++k)                // 16 keys per MMA: 8 columns of packed P, 32 bytes of a V^T row
                        mma_ts(tmem + O_COL0 + 128 * h, tmem + SP_COL0 + AT_STEP_KEYS * (j & 1) + 64 * h + 8 * k,
                               v_desc + ((h * V_BYTES + k * 32) >> 4), idesc_o, begun[h] || k != 0);
                    begun[h] = true;
                }
                if (!ok) break;
                mma_commit(&kv_empty[s]);              // the step's P V has ended: its stage is free, its O may be read
            }
        }
    } else {
        // Softmax: thread (quarter, lane) of half h has query row 32 quarter + lane and page h of every step.  A wait that
        // gives up does not end the loop: the block's later waits then return at once, and every thread reaches the
        // barriers of the end.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;                   // the query row of this thread = its lane of tensor memory
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t o_mine = lane_base + O_COL0 + 128 * half;
        const bool valid = q0 + row < q_len;
        const int hi = valid ? start + q0 + row : -1;
        const int lo = (valid && p.window > 0) ? max(0, hi - p.window + 1) : 0;
        float m_used = -INFINITY, l_sum = 0.f;
        bool ok = true, begun = false;
        for (int j = 0; j < num_steps; ++j) {
            if (half >= num_pages - AT_STEP_PAGES * j) break;  // the last step may have one page
            if (!bar_wait(&s_full[j & 1], (j >> 1) & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 16); ok = false; }
            fence_after_sync();
            const uint32_t mine = lane_base + SP_COL0 + AT_STEP_KEYS * (j & 1) + FRB_PAGE * half;
            const int key0 = (first_page + AT_STEP_PAGES * j + half) * FRB_PAGE;
            uint32_t raw[FRB_PAGE / 16][16];
#pragma unroll
            for (int c = 0; c < FRB_PAGE / 16; ++c) tmem_ld16(mine + 16 * c, raw[c]);
            tmem_wait_ld();
            // Most pages lie wholly before the tile's first query (and inside the window): no key of theirs is
            // masked for any row of this warp, and the per-key comparisons are left out.
            const bool open_page = __all_sync(0xffffffffu, valid && key0 + FRB_PAGE - 1 <= hi && key0 >= lo);
            float step_max;
            if (open_page) {
                float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains: a single one waits on itself
#pragma unroll
                for (int c = 0; c < FRB_PAGE / 16; ++c)
#pragma unroll
                    for (int i = 0; i < 16; i += 2)
                        top[(i >> 1) & 3] = max3(top[(i >> 1) & 3], __uint_as_float(raw[c][i]), __uint_as_float(raw[c][i + 1]));
                step_max = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3])) * p.scale2;     // the scale is positive
            } else {
                step_max = -INFINITY;
#pragma unroll
                for (int c = 0; c < FRB_PAGE / 16; ++c)
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int key = key0 + 16 * c + i;
                        const float v = key >= lo && key <= hi ? __uint_as_float(raw[c][i]) : -INFINITY;
                        raw[c][i] = __float_as_uint(v);
                        step_max = fmaxf(step_max, v * p.scale2);
                    }
            }
            float corr = 1.f;
            const bool raise = step_max > m_used + AT_RAISE;   // also true on the first page with a visible key
            if (raise) { corr = exp2f(m_used - step_max); m_used = step_max; }
            const float m_sub = m_used == -INFINITY ? 0.f : m_used;
            // 2^(s * scale - m) for two keys at a time: one multiply-add on the pair, the hardware's exponential on each
            // (a masked key gives 2^-inf = 0), one addition of the pair into one of four running pairs of sums.  (The
            // softmax is bound by the instructions it issues: a cubic on the multiply-add pipe for part of the
            // exponentials, to spare the special-function unit, made the kernel slower.)
            const uint64_t scale_pair = pair_of(p.scale2, p.scale2), shift_pair = pair_of(-m_sub, -m_sub);
            uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};
            uint32_t packed[FRB_PAGE / 32][16];
#pragma unroll
            for (int c = 0; c < FRB_PAGE / 16; ++c)
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float x0, x1;
                    halves_of(fma_pairs(pair_of(__uint_as_float(raw[c][i]), __uint_as_float(raw[c][i + 1])), scale_pair, shift_pair), x0, x1);
                    const float a = exp2_fast(x0), bb = exp2_fast(x1);
                    sums[(i >> 1) & 3] = add_pairs(sums[(i >> 1) & 3], pair_of(a, bb));
                    packed[c >> 1][(c & 1) * 8 + (i >> 1)] = pack_bf16x2(a, bb);
                }
            float sum_even, sum_odd;
            halves_of(add_pairs(add_pairs(sums[0], sums[1]), add_pairs(sums[2], sums[3])), sum_even, sum_odd);
            l_sum = l_sum * corr + (sum_even + sum_odd);
            if (begun && __any_sync(0xffffffffu, raise)) {     // rare: this page's O must follow the new maximum
                if (!bar_wait(&kv_empty[(j - 1) % AT_STAGES], ((j - 1) / AT_STAGES) & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 18); ok = false; }
                fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < HD / 16; ++c) {
                    uint32_t o[16];
                    tmem_ld16(o_mine + 16 * c, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st16(o_mine + 16 * c, o);
                }
            }
            begun = true;
            // P goes over the first half of the columns that this thread's scores came from
#pragma unroll
            for (int c = 0; c < FRB_PAGE / 32; ++c) tmem_st16(mine + 16 * c, packed[c]);
            tmem_wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) bar_arrive(&p_full[j & 1][half]);
        }
        {
            // A wait names a phase by its parity only, so it may not be two phases ahead of its barrier.  A thread whose
            // page the last step did not have comes here a step early: it waits for the step before the last first
            // (its own last one), after which the last step's barrier is at most one phase behind.
            const int last = num_steps - 1;
            if (last > 0 && !bar_wait(&kv_empty[(last - 1) % AT_STAGES], ((last - 1) / AT_STAGES) & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 19); ok = false; }
            if (!bar_wait(&kv_empty[last % AT_STAGES], (last / AT_STAGES) & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 19); ok = false; }
            fence_after_sync();
        }
        // The two threads of a row tell each other their maximum and sum (the stages of keys and values are free now:
        // every MMA has ended), then each writes half of the row's output from both accumulators.
        float* told = reinterpret_cast<float*>(stage0);        // [2 halves][128 rows][m, l]
        told[(half * AT_QUERIES + row) * 2] = m_used;
        told[(half * AT_QUERIES + row) * 2 + 1] = l_sum;
        asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX_THREADS) : "memory");
        const float m_other = told[((half ^ 1) * AT_QUERIES + row) * 2], l_other = told[((half ^ 1) * AT_QUERIES + row) * 2 + 1];
        const float m_both = fmaxf(m_used, m_other);
        const float a_mine = m_used == -INFINITY ? 0.f : exp2f(m_used - m_both);
        const float a_other = m_other == -INFINITY ? 0.f : exp2f(m_other - m_both);
        const float l_both = l_sum * a_mine + l_other * a_other;
        const float inv = l_both > 0.f ? 1.0f / l_both : 0.f;
        // O_1 holds nothing if every step had one page (a sequence of at most 64 keys in reach)
        const float w0 = (half == 0 ? a_mine : a_other) * inv, w1 = num_pages > 1 ? (half == 0 ? a_other : a_mine) * inv : 0.f;
        if (ok && !*failed) {
            constexpr int MINE = HD / 2;                       // output columns of this thread: [MINE half, MINE half + MINE)
            bf16* dst = p.out + ((size_t)(tok0 + row) * p.num_heads + head) * HD + MINE * half;
#pragma unroll 1
            for (int c = 0; c < MINE / 16; ++c) {
                uint32_t o0[16], o1[16];
                tmem_ld16(lane_base + O_COL0 + MINE * half + 16 * c, o0);
                if (num_pages > 1) tmem_ld16(lane_base + O_COL0 + 128 + MINE * half + 16 * c, o1);
                tmem_wait_ld();
                if (valid) {
                    float y[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        y[i] = __uint_as_float(o0[i]) * w0;
                        if (num_pages > 1) y[i] = fmaf(__uint_as_float(o1[i]), w1, y[i]);
                    }
                    uint4 lo4, hi4;
                    lo4.x = pack_bf16x2(y[0], y[1]);   lo4.y = pack_bf16x2(y[2], y[3]);
                    lo4.z = pack_bf16x2(y[4], y[5]);   lo4.w = pack_bf16x2(y[6], y[7]);
                    hi4.x = pack_bf16x2(y[8], y[9]);   hi4.y = pack_bf16x2(y[10], y[11]);
                    hi4.z = pack_bf16x2(y[12], y[13]); hi4.w = pack_bf16x2(y[14], y[15]);
                    reinterpret_cast<uint4*>(dst + 16 * c)[0] = lo4;
                    reinterpret_cast<uint4*>(dst + 16 * c)[1] = hi4;
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (failed_flag && warp == 0 && lane == 0) {
        // copies may still be on their way into this block's shared memory: give them a bounded time to land
        int zero = 0;
        bar_wait(&q_full, 0, &zero);
        for (int s = 0; s < AT_STAGES; ++s) { zero = 0; bar_wait(&kv_full[s], 0, &zero); }
    }
    __syncthreads();
    if (warp == 1) tmem_free(tmem, TMEM_COLS);
}

// ----------------------------------------------------------------------------- host side

// q bf16 [num_tokens, nh, hd]; k_pages [pages, nkv, 64, hd]; v_pages [pages, nkv, hd, 64]; tiles of 128 queries.
// status: one int on the device, zero before the call.
FRB_API int frb_attention_prefill_tc(const void* q, int num_tokens, const void* k_pages, const void* v_pages, int num_pages,
                                     const int* page_table, int max_pages, const int* tile_seq, const int* tile_q0,
                                     int num_tiles, const int* seq_slot, const int* seq_start, const int* seq_q_len,
                                     const int* cu_q_len, void* out, int num_heads, int num_kv_heads, int head_dim, float scale,
                                     int window, int* status, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    FRB_CHECK_ARG(head_dim == 64 || head_dim == 128, "tensor-core attention: head_dim %d is neither 64 nor 128", head_dim);
    FRB_CHECK_ARG(scale > 0.f, "tensor-core attention: a softmax scale of %g is not positive", (double)scale);
    FRB_CHECK_ARG(num_kv_heads > 0 && num_heads % num_kv_heads == 0 && num_heads <= 65535, "tensor-core attention: %d heads over %d kv heads",
                  num_heads, num_kv_heads);
    CUtensorMap map_q, map_k, map_v;
    const uint64_t kv_rows = (uint64_t)num_pages * num_kv_heads;
    FRB_CHECK_ARG(map_rows_of_64(&map_q, q, num_tokens, (uint64_t)num_heads * head_dim, AT_QUERIES) &&
                  map_rows_of_64(&map_k, k_pages, kv_rows * FRB_PAGE, head_dim, FRB_PAGE) &&
                  map_rows_of_64(&map_v, v_pages, kv_rows * head_dim, FRB_PAGE, head_dim),
                  "tensor-core attention: cuTensorMapEncodeTiled failed or is not available");
    AttnTcParams p;
    p.page_table = page_table; p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.seq_slot = seq_slot; p.seq_start = seq_start;
    p.seq_q_len = seq_q_len; p.cu_q_len = cu_q_len; p.out = (bf16*)out; p.status = status;
    p.scale2 = scale * 1.4426950408889634f; p.window = window; p.max_pages = max_pages; p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads;
    const size_t smem = (size_t)AT_QUERIES * head_dim * 2 + (size_t)AT_STAGES * AT_STEP_PAGES * 2 * FRB_PAGE * head_dim * 2 + 1024;
    dim3 grid(num_tiles, num_heads);
    if (head_dim == 128) {
        cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(attention_prefill_tc_kernel<128>, grid, dim3(AT_THREADS), smem, stream, map_q, map_k, map_v, p);
    } else {
        cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(attention_prefill_tc_kernel<64>, grid, dim3(AT_THREADS), smem, stream, map_q, map_k, map_v, p);
    }
    FRB_RETURN_LAUNCH("attention_prefill_tc");
}
