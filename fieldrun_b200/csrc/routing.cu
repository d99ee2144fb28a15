// Routing of tokens to experts: scores and top-k choice, the expert-sorted work lists that the expert
// products run over, and the weighted sum of the experts' outputs.
//
// Router (src/minimax.rs:94-104): s_e = 1/(1+exp(-z_e)); choice c_e = s_e + bias_e; experts in descending c,
// a tie going to the lower id (the reference sorts stably); the first k; weight w_e = s_e / sum of the
// picked s.  The bias enters the choice only.  Combination (src/minimax.rs:121-123): out[t] = sum over the
// picked experts of w * y; here always in rank order, so the sum does not depend on the batch.
#include "common.cuh"

// ----------------------------------------------------------------------------- top-k choice

// Floats as unsigned integers in the same order (so that the warp's maximum is one redux instruction).
__device__ __forceinline__ unsigned int ordered_bits(float v) {
    const unsigned int u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

#define PICK_PER_LANE 8      // experts a lane keeps in registers: up to 256 experts on the fast path

// One warp picks one token's experts.  z: the token's E logits; score/choice: E floats of scratch each.
// Each lane owns the experts lane, lane + 32, ...; a pass finds the largest choice value in the warp (ties:
// the lowest expert id, as a stable sort would), hands it out and removes it.
__device__ __forceinline__ void pick_experts(const float* __restrict__ z, const float* __restrict__ bias, int num_experts,
                                             int top_k, int renormalize, float routed_scale, float* score, float* choice,
                                             int* __restrict__ ids, float* __restrict__ weights, int lane) {
    float denom = 0.f;
    if (num_experts <= 32 * PICK_PER_LANE && top_k <= 32) {
        // the lane's candidates stay in registers; NaN scores count as the smallest value
        float mine[PICK_PER_LANE], sc[PICK_PER_LANE];
        // every load goes out before the first value is used (inside the branches below they went one after the
        // other, each waiting for L2: 5 to 6 us of a decode step's router)
        float logit[PICK_PER_LANE], shift[PICK_PER_LANE];
#pragma unroll
        for (int i = 0; i < PICK_PER_LANE; ++i) {
            const int e = min(lane + 32 * i, num_experts - 1);
            logit[i] = __ldcg(z + e);                                    // read through L2: another block may have written it
            shift[i] = bias ? __ldg(bias + e) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < PICK_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < num_experts) {
                const float s = 1.0f / (1.0f + expf(-logit[i]));
                sc[i] = s;
                const float c = bias ? s + shift[i] : s;
                mine[i] = c == c ? c : -INFINITY;
            } else {
                sc[i] = 0.f;
                mine[i] = -INFINITY;
            }
        }
        unsigned int taken = 0;                         // bit i: this lane's candidate i is handed out (or absent)
#pragma unroll
        for (int i = 0; i < PICK_PER_LANE; ++i)
            if (lane + 32 * i >= num_experts) taken |= 1u << i;
        float picked_score = 0.f;                       // lane r keeps the score of the rank-r pick
        int picked_id = 0;
        for (int r = 0; r < top_k; ++r) {
            float best = -INFINITY;
            int best_i = -1;
#pragma unroll
            for (int i = 0; i < PICK_PER_LANE; ++i)
                if (!(taken & (1u << i)) && (best_i < 0 || mine[i] > best)) { best = mine[i]; best_i = i; }
            const unsigned int key = best_i >= 0 ? ordered_bits(best) : 0u;
            const unsigned int top = __reduce_max_sync(0xffffffffu, key);
            const int my_e = (best_i >= 0 && key == top) ? lane + 32 * best_i : 0x7fffffff;
            const int e = __reduce_min_sync(0xffffffffu, my_e);          // the lowest id among equal values
            const int owner = e & 31, slot = e >> 5;
            float s_e = 0.f;
#pragma unroll
            for (int i = 0; i < PICK_PER_LANE; ++i)
                if (i == slot) s_e = sc[i];
            s_e = __shfl_sync(0xffffffffu, s_e, owner);
            if (lane == owner) taken |= 1u << slot;
            if (lane == r) { picked_score = s_e; picked_id = e; }
            denom += s_e;
        }
        if (lane < top_k) {
            float w = picked_score;
            if (renormalize) w = w / denom;               // s_e / sum of picked s (src/minimax.rs:100-103)
            ids[lane] = picked_id;
            weights[lane] = w * routed_scale;
        }
        __syncwarp();
        return;
    }
    for (int e = lane; e < num_experts; e += 32) {
        const float s = 1.0f / (1.0f + expf(-__ldcg(z + e)));
        score[e] = s;
        choice[e] = bias ? s + bias[e] : s;
    }
    __syncwarp();
    for (int r = 0; r < top_k; ++r) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < num_experts; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; best_e = e; }      // ascending e: the first of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) {                       // nothing comparable is left (NaN scores): lowest unpicked id
            best_e = 0;
            while (best_e < num_experts - 1 && choice[best_e] == -INFINITY) ++best_e;
        }
        __syncwarp();
        if (lane == 0) {
            ids[r] = best_e;
            weights[r] = score[best_e];
            choice[best_e] = -INFINITY;
        }
        denom += score[best_e];
        __syncwarp();
    }
    if (lane == 0) {
        for (int r = 0; r < top_k; ++r) {
            float w = weights[r];
            if (renormalize) w = w / denom;               // s_e / sum of picked s (src/minimax.rs:100-103)
            weights[r] = w * routed_scale;
        }
    }
    __syncwarp();
}

// One warp per token.  logits [T, E] float32 -> ids [T, k] (rank order), weights [T, k].
__global__ void router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int num_experts,
                                   int top_k, int renormalize, float routed_scale, int* __restrict__ ids,
                                   float* __restrict__ weights) {
    after_previous_kernel();
    extern __shared__ float sm[];
    const int t = blockIdx.x;
    pick_experts(logits + (size_t)t * num_experts, bias, num_experts, top_k, renormalize, routed_scale, sm, sm + num_experts,
                 ids + (size_t)t * top_k, weights + (size_t)t * top_k, threadIdx.x);
}

FRB_API int frb_router_topk(const float* logits, const float* bias, int num_tokens, int num_experts, int top_k,
                            int renormalize, float routed_scale, int* ids, float* weights, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(top_k >= 1 && top_k <= num_experts, "router: top_k %d is outside 1..%d experts", top_k, num_experts);
    const size_t smem = (size_t)2 * num_experts * sizeof(float);
    FRB_CHECK_ARG(smem <= 48 * 1024, "router: %d experts exceed the kernel's 6144", num_experts);
    launch_dependent(router_topk_kernel, dim3(num_tokens), dim3(32), smem, stream, logits, bias, num_experts, top_k, renormalize, routed_scale, ids,
                                                         weights);
    FRB_RETURN_LAUNCH("router_topk");
}

// ----------------------------------------------------------------------------- expert-sorted work lists

#define PLAN_CHUNK 1024     // assignments per block
#define PLAN_BLOCK 256

// counts[c][e] = number of assignments of chunk c that go to expert e
__global__ void __launch_bounds__(PLAN_BLOCK)
plan_count_kernel(const int* __restrict__ ids, int num_assign, int num_experts, int* __restrict__ counts) {
    extern __shared__ int hist[];
    const int c = blockIdx.x;
    let_next_kernel_start();
    for (int e = threadIdx.x; e < num_experts; e += PLAN_BLOCK) hist[e] = 0;
    wait_for_previous_kernel();
    __syncthreads();
    const int begin = c * PLAN_CHUNK, end = min(num_assign, begin + PLAN_CHUNK);
    for (int a = begin + threadIdx.x; a < end; a += PLAN_BLOCK) atomicAdd(&hist[ids[a]], 1);
    __syncthreads();
    for (int e = threadIdx.x; e < num_experts; e += PLAN_BLOCK) counts[(size_t)c * num_experts + e] = hist[e];
}

// Turns counts into starting positions: counts[c][e] becomes the place of chunk c's first assignment to e;
// offsets[e] the first row of expert e in the sorted list; tiles of `tile_rows` rows that never span two
// experts are listed in (tile_expert, tile_row0) and counted in num_tiles[0].
__global__ void __launch_bounds__(PLAN_BLOCK)
plan_scan_kernel(int* __restrict__ counts, int num_chunks, int num_experts, int tile_rows, int* __restrict__ offsets,
                 int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ num_tiles) {
    after_previous_kernel();
    extern __shared__ int total[];       // [E] totals, then [E + 1] first rows, then [E + 1] first tiles
    int* first = total + num_experts;
    int* first_tile = first + num_experts + 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < num_experts; e += PLAN_BLOCK) {
        int run = 0;
        for (int c = 0; c < num_chunks; ++c) {
            const int n = counts[(size_t)c * num_experts + e];
            counts[(size_t)c * num_experts + e] = run;
            run += n;
        }
        total[e] = run;
    }
    __syncthreads();
    if (warp == 0) {                     // exclusive sums over the experts: each lane a run of experts, then a warp scan
        const int per_lane = (num_experts + 31) / 32;
        const int begin = lane * per_lane, end = min(num_experts, begin + per_lane);
        int rows = 0, tiles = 0;
        for (int e = begin; e < end; ++e) { rows += total[e]; tiles += (total[e] + tile_rows - 1) / tile_rows; }
        int rows_before = rows, tiles_before = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int r = __shfl_up_sync(0xffffffffu, rows_before, o), c = __shfl_up_sync(0xffffffffu, tiles_before, o);
            if (lane >= o) { rows_before += r; tiles_before += c; }
        }
        const int all_rows = __shfl_sync(0xffffffffu, rows_before, 31), all_tiles = __shfl_sync(0xffffffffu, tiles_before, 31);
        rows_before -= rows;
        tiles_before -= tiles;
        for (int e = begin; e < end; ++e) {
            first[e] = rows_before;
            first_tile[e] = tiles_before;
            rows_before += total[e];
            tiles_before += (total[e] + tile_rows - 1) / tile_rows;
        }
        if (lane == 0) { first[num_experts] = all_rows; num_tiles[0] = all_tiles; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= num_experts; e += PLAN_BLOCK) offsets[e] = first[e];
    for (int e = threadIdx.x; e < num_experts; e += PLAN_BLOCK) {
        int tile = first_tile[e];
        for (int r = 0; r < total[e]; r += tile_rows, ++tile) {
            tile_expert[tile] = e;
            tile_row0[tile] = first[e] + r;
        }
        for (int c = 0; c < num_chunks; ++c) counts[(size_t)c * num_experts + e] += first[e];
    }
}

// Places every assignment a = t*k + r, in order, behind the earlier ones of the same expert.  One warp walks
// the chunk 32 assignments at a time: lanes with the same expert find one another with a match, take
// consecutive places from the expert's running counter, and the lowest of them moves the counter on.
__global__ void __launch_bounds__(PLAN_BLOCK)
plan_fill_kernel(const int* __restrict__ ids, int num_assign, int num_experts, int top_k, const int* __restrict__ counts,
                 int* __restrict__ sorted_token, int* __restrict__ row_of_assign) {
    after_previous_kernel();
    extern __shared__ int next_place[];          // [E]
    __shared__ int place[PLAN_CHUNK];            // first the chunk's expert ids (all threads fetch them), then their places
    const int c = blockIdx.x;
    const int begin = c * PLAN_CHUNK, n = min(num_assign - begin, PLAN_CHUNK);
    for (int e = threadIdx.x; e < num_experts; e += PLAN_BLOCK) next_place[e] = counts[(size_t)c * num_experts + e];
    for (int i = threadIdx.x; i < n; i += PLAN_BLOCK) place[i] = ids[begin + i];
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        for (int base = 0; base < n; base += 32) {
            const int i = base + lane;
            const bool live = i < n;
            const int e = live ? place[i] : -1 - lane;                   // idle lanes match nobody
            const unsigned same = __match_any_sync(0xffffffffu, e);
            const int rank = __popc(same & ((1u << lane) - 1));
            if (live) place[i] = next_place[e] + rank;
            __syncwarp();
            if (live && rank == 0) next_place[e] += __popc(same);
            __syncwarp();
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += PLAN_BLOCK) {
        const int a = begin + i;
        sorted_token[place[i]] = a / top_k;
        row_of_assign[a] = place[i];
    }
}

// ids [T, k] -> offsets [E+1], sorted_token [N], row_of_assign [N], tiles.  `counts` is scratch of
// ceil(N / 1024) * E ints.  Tile lists need room for ceil(N / tile_rows) + min(E, N) entries.
FRB_API int frb_expert_plan(const int* ids, int num_tokens, int top_k, int num_experts, int tile_rows, int* counts,
                            int* offsets, int* sorted_token, int* row_of_assign, int* tile_expert, int* tile_row0,
                            int* num_tiles, cudaStream_t stream) {
    const int num_assign = num_tokens * top_k;
    if (num_assign == 0) return 0;
    FRB_CHECK_ARG((3 * num_experts + 2) * sizeof(int) <= 48 * 1024, "expert plan: %d experts exceed the kernel's 4095", num_experts);
    const int chunks = (num_assign + PLAN_CHUNK - 1) / PLAN_CHUNK;
    const size_t smem = (size_t)num_experts * sizeof(int);
    launch_dependent(plan_count_kernel, dim3(chunks), dim3(PLAN_BLOCK), smem, stream, ids, num_assign, num_experts, counts);
    launch_dependent(plan_scan_kernel, dim3(1), dim3(PLAN_BLOCK), 3 * smem + 2 * sizeof(int), stream, counts, chunks, num_experts,
                     tile_rows, offsets, tile_expert, tile_row0, num_tiles);
    launch_dependent(plan_fill_kernel, dim3(chunks), dim3(PLAN_BLOCK), smem, stream, ids, num_assign, num_experts, top_k,
                     (const int*)counts, sorted_token, row_of_assign);
    FRB_RETURN_LAUNCH("expert_plan");
}

// ----------------------------------------------------------------------------- choice and work lists in one block

#define SMALL_WARPS 16
#define SMALL_MAX_ASSIGN 1024

// For steps of few tokens (T * k <= 1024): one block picks every token's experts (a warp per token, in
// turn), then sorts the assignments by expert and writes the same lists as the three kernels above.
struct SmallRouteParams {
    const float* logits;     // [T, E]
    const float* bias;       // [E] or null
    int num_tokens, num_experts, top_k, renormalize;
    float routed_scale;
    int tile_rows;
    int* ids;                // [T, k]
    float* weights;          // [T, k]
    int* offsets;            // [E + 1]
    int* sorted_token;       // [N]
    int* row_of_assign;      // [N]
    int* tile_expert;
    int* tile_row0;
    int* num_tiles;
};

#define TINY_MAX_ASSIGN 128      // up to this many (token, expert) pairs the lists are made without counting over the experts

// The lists for a handful of assignments (a decode step of a few sequences), with one barrier: every thread
// finds what it has to write by looking through all assignments in shared memory, n^2 comparisons in all.
// Assignment a lies behind the assignments of lower experts and the earlier ones of its own expert (the order
// of the counting sort); the first assignment of an expert writes the expert's tiles.
__device__ __forceinline__ void plan_tiny(const SmallRouteParams& p, const int* s_ids, int* s_tiles) {
    const int n = p.num_tokens * p.top_k, tile_rows = p.tile_rows;
    for (int e = threadIdx.x; e <= p.num_experts; e += blockDim.x) {
        int before = 0;
        for (int b = 0; b < n; ++b) before += s_ids[b] < e;
        p.offsets[e] = before;
    }
    // every assignment's place; the first assignment of an expert notes how many tiles the expert has
    int lower = 0, earlier = 0, same = 0;                     // of assignment threadIdx.x (n <= blockDim.x)
    const int a = threadIdx.x, e = a < n ? s_ids[a] : 0;
    if (a < n) {
        for (int b = 0; b < n; ++b) {
            const int eb = s_ids[b];
            lower += eb < e;
            same += eb == e;
            earlier += eb == e && b < a;
        }
        p.sorted_token[lower + earlier] = a / p.top_k;
        p.row_of_assign[a] = lower + earlier;
        s_tiles[a] = earlier == 0 ? (same + tile_rows - 1) / tile_rows : 0;
    }
    __syncthreads();
    if (a < n && earlier == 0) {
        int tile = 0;                                         // tiles of the experts before this one
        for (int b = 0; b < n; ++b) tile += s_ids[b] < e ? s_tiles[b] : 0;
        for (int r = 0; r < same; r += tile_rows, ++tile) {
            p.tile_expert[tile] = e;
            p.tile_row0[tile] = lower + r;
        }
        if (lower + same == n) p.num_tiles[0] = tile;         // the highest expert in use ends the list
    }
}

// The work of one block of SMALL_WARPS warps: every token's choice, then the lists.  sm: dynamic shared memory.
__device__ __forceinline__ void route_and_plan(const SmallRouteParams& p, float* sm, int* s_ids) {
    const int num_experts = p.num_experts, top_k = p.top_k, tile_rows = p.tile_rows;
    if (p.num_tokens * top_k <= TINY_MAX_ASSIGN && p.num_tokens <= SMALL_WARPS && top_k <= 32) {
        // a warp per token picks; the picks go to shared memory as well, for the lists
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (warp < p.num_tokens) {
            pick_experts(p.logits + (size_t)warp * num_experts, p.bias, num_experts, top_k, p.renormalize, p.routed_scale,
                         sm + (size_t)warp * 2 * num_experts, sm + (size_t)warp * 2 * num_experts + num_experts,
                         p.ids + (size_t)warp * top_k, p.weights + (size_t)warp * top_k, lane);
            if (lane < top_k) s_ids[warp * top_k + lane] = p.ids[warp * top_k + lane];      // written by this warp, above
        }
        __syncthreads();
        plan_tiny(p, s_ids, reinterpret_cast<int*>(sm));      // the picks' scratch is free now
        return;
    }
    float* scratch = sm;                                                 // [SMALL_WARPS][2][E]
    int* count = reinterpret_cast<int*>(sm + (size_t)SMALL_WARPS * 2 * num_experts);   // [E]
    int* first = count + num_experts;                                    // [E + 1]
    int* first_tile = first + num_experts + 1;                           // [E + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int num_assign = p.num_tokens * top_k;
    for (int t = warp; t < p.num_tokens; t += SMALL_WARPS)
        pick_experts(p.logits + (size_t)t * num_experts, p.bias, num_experts, top_k, p.renormalize, p.routed_scale,
                     scratch + (size_t)warp * 2 * num_experts, scratch + (size_t)warp * 2 * num_experts + num_experts,
                     p.ids + (size_t)t * top_k, p.weights + (size_t)t * top_k, lane);
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < num_assign; a += blockDim.x) {
        const int e = p.ids[a];                                          // written by this block, above
        s_ids[a] = e;
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (warp == 0) {                                                     // exclusive sums over the experts
        const int per_lane = (num_experts + 31) / 32;
        const int begin = lane * per_lane, end = min(num_experts, begin + per_lane);
        int rows = 0, tiles = 0;
        for (int e = begin; e < end; ++e) { rows += count[e]; tiles += (count[e] + tile_rows - 1) / tile_rows; }
        int rows_before = rows, tiles_before = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int r = __shfl_up_sync(0xffffffffu, rows_before, o), c = __shfl_up_sync(0xffffffffu, tiles_before, o);
            if (lane >= o) { rows_before += r; tiles_before += c; }
        }
        const int total_rows = __shfl_sync(0xffffffffu, rows_before, 31), total_tiles = __shfl_sync(0xffffffffu, tiles_before, 31);
        rows_before -= rows;
        tiles_before -= tiles;
        for (int e = begin; e < end; ++e) {
            first[e] = rows_before;
            first_tile[e] = tiles_before;
            rows_before += count[e];
            tiles_before += (count[e] + tile_rows - 1) / tile_rows;
        }
        if (lane == 0) { first[num_experts] = total_rows; p.num_tiles[0] = total_tiles; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= num_experts; e += blockDim.x) p.offsets[e] = first[e];
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        int tile = first_tile[e];
        for (int r = 0; r < count[e]; r += tile_rows, ++tile) {
            p.tile_expert[tile] = e;
            p.tile_row0[tile] = first[e] + r;
        }
    }
    __syncthreads();                                                     // first[] is read above and moved below
    if (warp == 0) {
        // one warp walks the assignments 32 at a time, in order: lanes with the same expert find one another
        // with a match and take consecutive places behind the expert's earlier rows (first[] moves on)
        for (int base = 0; base < num_assign; base += 32) {
            const int a = base + lane;
            const bool live = a < num_assign;
            const int e = live ? s_ids[a] : -1 - lane;
            const unsigned same = __match_any_sync(0xffffffffu, e);
            const int rank = __popc(same & ((1u << lane) - 1));
            int at = 0;
            if (live) at = first[e] + rank;
            __syncwarp();
            if (live && rank == 0) first[e] += __popc(same);
            __syncwarp();
            if (live) {
                p.sorted_token[at] = a / top_k;
                p.row_of_assign[a] = at;
            }
        }
    }
}

__global__ void __launch_bounds__(SMALL_WARPS * 32) route_plan_small_kernel(SmallRouteParams p) {
    after_previous_kernel();
    extern __shared__ float sm[];
    __shared__ int s_ids[SMALL_MAX_ASSIGN];
    route_and_plan(p, sm, s_ids);
}

#define ROUTER_SMALL_TOKENS 8       // most tokens of a step that the one-launch router takes
#define ROUTER_SMALL_EXPERTS 2      // experts per block: SMALL_WARPS / 2 warps share one expert's inner size
#define ROUTER_EARLY 4              // 16-byte loads of the router's weight that a lane sends ahead of the wait (widths to 4096)

// Router logits and everything after them in one launch, for steps of at most 8 tokens.  A block computes
// the logits of two experts: eight warps each take an eighth of an expert's float32 weight row against
// every token's float32 row; their partial sums are added in warp order.  The block that finishes last then
// picks the experts and makes the lists.
__global__ void __launch_bounds__(SMALL_WARPS * 32)
router_small_kernel(const float* __restrict__ act, const float* __restrict__ router, int width, float* __restrict__ logits,
                    unsigned int* __restrict__ ticket, SmallRouteParams p) {
    extern __shared__ float sm[];
    __shared__ int s_ids[SMALL_MAX_ASSIGN];
    __shared__ float s_part[SMALL_WARPS][ROUTER_SMALL_TOKENS];
    __shared__ int s_last;
    constexpr int WARPS_PER_EXPERT = SMALL_WARPS / ROUTER_SMALL_EXPERTS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.x * ROUTER_SMALL_EXPERTS + warp / WARPS_PER_EXPERT;
    const int part = warp % WARPS_PER_EXPERT;
    const int vecs = width / 4;
    const int per_part = (vecs + WARPS_PER_EXPERT - 1) / WARPS_PER_EXPERT;
    const int begin = part * per_part, end = min(vecs, begin + per_part);
    const float4* w = reinterpret_cast<const float4*>(router + (size_t)min(e, p.num_experts - 1) * width);
    // the router's weight does not wait for the kernel before this one: its first loads go out ahead of the wait
    let_next_kernel_start();
    float4 early[ROUTER_EARLY];
#pragma unroll
    for (int i = 0; i < ROUTER_EARLY; ++i)
        if (begin + lane + 32 * i < end) early[i] = __ldg(w + begin + lane + 32 * i);
    wait_for_previous_kernel();
    float acc[ROUTER_SMALL_TOKENS];
#pragma unroll
    for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j) acc[j] = 0.f;
    if (e < p.num_experts) {
#pragma unroll
        for (int i = 0; i < ROUTER_EARLY; ++i) {
            const int k = begin + lane + 32 * i;
            if (k < end) {
                float4 xv[ROUTER_SMALL_TOKENS];                  // every token's loads go out before the first is used
#pragma unroll
                for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j)
                    xv[j] = __ldg(reinterpret_cast<const float4*>(act + (size_t)min(j, p.num_tokens - 1) * width) + k);
#pragma unroll
                for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j)
                    if (j < p.num_tokens)
                        acc[j] += xv[j].x * early[i].x + xv[j].y * early[i].y + xv[j].z * early[i].z + xv[j].w * early[i].w;
            }
        }
        for (int k = begin + lane + 32 * ROUTER_EARLY; k < end; k += 32) {
            const float4 wv = __ldg(w + k);
#pragma unroll
            for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j) {
                if (j < p.num_tokens) {
                    const float4 xv = __ldg(reinterpret_cast<const float4*>(act + (size_t)j * width) + k);
                    acc[j] += xv.x * wv.x + xv.y * wv.y + xv.z * wv.z + xv.w * wv.w;
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j) {
        const float total = warp_sum(acc[j]);
        if (lane == 0) s_part[warp][j] = total;
    }
    __syncthreads();
    if (threadIdx.x < ROUTER_SMALL_EXPERTS * ROUTER_SMALL_TOKENS) {
        const int local = threadIdx.x / ROUTER_SMALL_TOKENS, j = threadIdx.x % ROUTER_SMALL_TOKENS;
        const int expert = blockIdx.x * ROUTER_SMALL_EXPERTS + local;
        if (expert < p.num_experts && j < p.num_tokens) {
            float total = 0.f;
            for (int w = 0; w < WARPS_PER_EXPERT; ++w) total += s_part[local * WARPS_PER_EXPERT + w][j];
            logits[(size_t)j * p.num_experts + expert] = total;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int before = atomicAdd(ticket, 1u);
        s_last = before == gridDim.x - 1;
        if (s_last) *ticket = 0;                          // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    route_and_plan(p, sm, s_ids);
}

// Router logits alone, for steps of up to a few hundred tokens: a block computes the logits of two experts
// for eight tokens, in the same way (and the same order of additions) as router_small_kernel.  The library's
// float32 product takes 36 us for 64 tokens of MiniMax-M2's router (a split inner size on 28 blocks).
__global__ void __launch_bounds__(SMALL_WARPS * 32)
router_logits_kernel(const float* __restrict__ act, const float* __restrict__ router, int width, int num_tokens, int num_experts,
                     float* __restrict__ logits) {
    after_previous_kernel();
    __shared__ float s_part[SMALL_WARPS][ROUTER_SMALL_TOKENS];
    constexpr int WARPS_PER_EXPERT = SMALL_WARPS / ROUTER_SMALL_EXPERTS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.x * ROUTER_SMALL_EXPERTS + warp / WARPS_PER_EXPERT;
    const int part = warp % WARPS_PER_EXPERT;
    const int token0 = blockIdx.y * ROUTER_SMALL_TOKENS, tokens = min(ROUTER_SMALL_TOKENS, num_tokens - token0);
    float acc[ROUTER_SMALL_TOKENS];
#pragma unroll
    for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j) acc[j] = 0.f;
    if (e < num_experts) {
        const int vecs = width / 4;
        const int per_part = (vecs + WARPS_PER_EXPERT - 1) / WARPS_PER_EXPERT;
        const int begin = part * per_part, end = min(vecs, begin + per_part);
        const float4* w = reinterpret_cast<const float4*>(router + (size_t)e * width);
        for (int k = begin + lane; k < end; k += 32) {
            const float4 wv = __ldg(w + k);
#pragma unroll
            for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j) {
                if (j < tokens) {
                    const float4 xv = __ldg(reinterpret_cast<const float4*>(act + (size_t)(token0 + j) * width) + k);
                    acc[j] += xv.x * wv.x + xv.y * wv.y + xv.z * wv.z + xv.w * wv.w;
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < ROUTER_SMALL_TOKENS; ++j) {
        const float total = warp_sum(acc[j]);
        if (lane == 0) s_part[warp][j] = total;
    }
    __syncthreads();
    if (threadIdx.x < ROUTER_SMALL_EXPERTS * ROUTER_SMALL_TOKENS) {
        const int local = threadIdx.x / ROUTER_SMALL_TOKENS, j = threadIdx.x % ROUTER_SMALL_TOKENS;
        const int expert = blockIdx.x * ROUTER_SMALL_EXPERTS + local;
        if (expert < num_experts && j < tokens) {
            float total = 0.f;
            for (int w = 0; w < WARPS_PER_EXPERT; ++w) total += s_part[local * WARPS_PER_EXPERT + w][j];
            logits[(size_t)(token0 + j) * num_experts + expert] = total;
        }
    }
}

// act [T, width] float32 rows, router [E, width] float32 -> logits [T, E].
FRB_API int frb_router_logits(const float* act, const float* router, int width, int num_tokens, int num_experts, float* logits,
                              cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(width % 4 == 0 && ((uintptr_t)act & 15) == 0 && ((uintptr_t)router & 15) == 0,
                  "router logits: a width of %d (or an unaligned operand) does not allow 16-byte loads", width);
    dim3 grid((num_experts + ROUTER_SMALL_EXPERTS - 1) / ROUTER_SMALL_EXPERTS, (num_tokens + ROUTER_SMALL_TOKENS - 1) / ROUTER_SMALL_TOKENS);
    FRB_CHECK_ARG(grid.y <= 65535, "router logits: %d tokens exceed the grid", num_tokens);
    launch_dependent(router_logits_kernel, grid, dim3(SMALL_WARPS * 32), 0, stream, act, router, width, num_tokens, num_experts, logits);
    FRB_RETURN_LAUNCH("router_logits");
}

static int small_route_params(SmallRouteParams& p, size_t& smem, const float* logits, const float* bias, int num_tokens,
                              int num_experts, int top_k, int renormalize, float routed_scale, int tile_rows, int* ids,
                              float* weights, int* offsets, int* sorted_token, int* row_of_assign, int* tile_expert,
                              int* tile_row0, int* num_tiles) {
    FRB_CHECK_ARG(top_k >= 1 && top_k <= num_experts, "router: top_k %d is outside 1..%d experts", top_k, num_experts);
    FRB_CHECK_ARG(num_tokens * top_k <= SMALL_MAX_ASSIGN, "small router: %d assignments exceed %d", num_tokens * top_k,
                  SMALL_MAX_ASSIGN);
    smem = (size_t)SMALL_WARPS * 2 * num_experts * sizeof(float) + (size_t)(3 * num_experts + 2) * sizeof(int);
    FRB_CHECK_ARG(smem <= 160 * 1024, "small router: %d experts need %zu bytes of shared memory", num_experts, smem);
    p.logits = logits; p.bias = bias; p.num_tokens = num_tokens; p.num_experts = num_experts; p.top_k = top_k;
    p.renormalize = renormalize; p.routed_scale = routed_scale; p.tile_rows = tile_rows; p.ids = ids; p.weights = weights;
    p.offsets = offsets; p.sorted_token = sorted_token; p.row_of_assign = row_of_assign; p.tile_expert = tile_expert;
    p.tile_row0 = tile_row0; p.num_tiles = num_tiles;
    return 0;
}

FRB_API int frb_route_plan_small(const float* logits, const float* bias, int num_tokens, int num_experts, int top_k,
                                 int renormalize, float routed_scale, int tile_rows, int* ids, float* weights, int* offsets,
                                 int* sorted_token, int* row_of_assign, int* tile_expert, int* tile_row0, int* num_tiles,
                                 cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    SmallRouteParams p;
    size_t smem;
    if (small_route_params(p, smem, logits, bias, num_tokens, num_experts, top_k, renormalize, routed_scale, tile_rows, ids,
                           weights, offsets, sorted_token, row_of_assign, tile_expert, tile_row0, num_tiles))
        return -1;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(route_plan_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_dependent(route_plan_small_kernel, dim3(1), dim3(SMALL_WARPS * 32), smem, stream, p);
    FRB_RETURN_LAUNCH("route_plan_small");
}

// act [T, width] float32 rows, router [E, width] float32 -> logits [T, E] (scratch, kept) and all of the above.
// ticket: one unsigned int on the device, zero before the first call (the kernel leaves it zero).
FRB_API int frb_router_small(const float* act, const float* router, int width, float* logits, unsigned int* ticket,
                             const float* bias, int num_tokens, int num_experts, int top_k, int renormalize,
                             float routed_scale, int tile_rows, int* ids, float* weights, int* offsets, int* sorted_token,
                             int* row_of_assign, int* tile_expert, int* tile_row0, int* num_tiles, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(width % 4 == 0 && ((uintptr_t)act & 15) == 0 && ((uintptr_t)router & 15) == 0,
                  "small router: a width of %d (or an unaligned operand) does not allow 16-byte loads", width);
    FRB_CHECK_ARG(num_tokens <= ROUTER_SMALL_TOKENS, "small router: %d tokens exceed %d", num_tokens, ROUTER_SMALL_TOKENS);
    SmallRouteParams p;
    size_t smem;
    if (small_route_params(p, smem, logits, bias, num_tokens, num_experts, top_k, renormalize, routed_scale, tile_rows, ids,
                           weights, offsets, sorted_token, row_of_assign, tile_expert, tile_row0, num_tiles))
        return -1;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(router_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int blocks = (num_experts + ROUTER_SMALL_EXPERTS - 1) / ROUTER_SMALL_EXPERTS;
    launch_dependent(router_small_kernel, dim3(blocks), dim3(SMALL_WARPS * 32), smem, stream, act, router, width, logits, ticket, p);
    FRB_RETURN_LAUNCH("router_small");
}

// ----------------------------------------------------------------------------- weighted sum of expert outputs

// out[t, :] = sum_{r < k} w[t, r] * y[row_of_assign[t*k + r], :], added in rank order.
__global__ void combine_kernel(const float* __restrict__ y, const float* __restrict__ weights,
                               const int* __restrict__ row_of_assign, int top_k, int width, float* __restrict__ out) {
    after_previous_kernel();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    float acc = 0.f;
    for (int r = 0; r < top_k; ++r) {
        const int row = row_of_assign[(size_t)t * top_k + r];
        acc += weights[(size_t)t * top_k + r] * y[(size_t)row * width + c];
    }
    out[(size_t)t * width + c] = acc;
}

FRB_API int frb_expert_combine(const float* y, const float* weights, const int* row_of_assign, int num_tokens, int top_k,
                               int width, float* out, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens, (width + 255) / 256);
    FRB_CHECK_ARG(grid.y <= 65535, "combine: a width of %d exceeds the grid", width);
    launch_dependent(combine_kernel, dim3(grid), dim3(256), 0, stream, y, weights, row_of_assign, top_k, width, out);
    FRB_RETURN_LAUNCH("expert_combine");
}
