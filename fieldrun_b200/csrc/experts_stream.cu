// Matrix products of a few rows with large bfloat16 weights, as one stream over the weights per SM.
//
// y[row, f] = sum_k x[row, k] W_e[f, k] for the rows routed to expert e (src/minimax.rs:116-120); a dense layer
// is a single "expert" whose rows are all the rows.  A decode step brings one or two rows per expert, so the
// weights are the traffic and the kernel is built around keeping them in flight:
//
//   * One block per SM for the whole launch.  The work is cut into items of sixteen weight rows over the whole
//     inner size (for a pair of matrices: eight gate rows and the eight up rows of the same features); block b
//     takes the b-th share of the items, one after another, so a block's set-up is paid once and the stream
//     never stops between items.
//   * A producer thread copies the items' weights with TMA into a ring of stages in shared memory (16 KB each:
//     sixteen rows x 512 k, as eight pieces of 64 k whose rows are 128 bytes, swizzled), always as far ahead as
//     the ring is long: about 100 KB in flight per SM whatever the compute warps are doing.  (Rows of 64 bytes
//     halve what the copy unit delivers: it works row by row, about 3.6 cycles each.)  Where the lists of tiles do not depend on the kernel before this one (a dense
//     layer; the second product of the experts, whose lists the first one used already), the ring is filled
//     before that kernel has ended: the launch is a programmatic dependent launch, and only the warps that read
//     x wait for it.
//   * Eight warps multiply: each takes one piece of every stage with mma.sync m16n8k16, the weights as the
//     16-row operand straight from shared memory (a thread's 16 bytes are 8 neighbouring k of one row, used for
//     two MMAs: the same regrouping of k on both operands, which a sum over k does not notice), the rows of x
//     as the 8-column operand from global memory through L1, asked for before the wait for the stage.  Row g of the operand is
//     weight row (g >> 1) + 4 (g & 1) of its run of eight: the two rows that a quarter of a warp reads then differ
//     in the bit that the swizzle moves to the other half of the 128 bytes, and no read meets a bank conflict.
//     At the end of an item the eight partial sums are added in the order of the warps, so a row's result does
//     not depend on what else the step holds.
//
// PAIRED: W = [E][2F][K] (gate rows then up rows); the epilogue writes silu(gate) * up as bfloat16.
// Otherwise W = [E][F][K] and the float32 products are written.
//
// Every wait on an mbarrier is bounded: a wait that runs out records a code in `status`, the block's other waits
// then return at once, nothing is stored, and the block leaves after the copies in flight have landed.
#include "tma.cuh"

using namespace frb_tma;

#define WS_COMPUTE_WARPS 8
#define WS_THREADS (32 * (WS_COMPUTE_WARPS + 1))
#define WS_MAX_STAGES 16
#define WS_PIECE_K 64                  // a piece: sixteen rows x 64 k x 2 bytes
#define WS_PIECE_BYTES 2048
#define WS_PER_WARP 3                  // pieces of a stage that one warp takes, at most
#define WS_MAX_PIECES (WS_PER_WARP * WS_COMPUTE_WARPS)   // pieces per stage: 1536 k, 48 KB

__device__ __forceinline__ void stream_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct StreamParams {
    const bf16* X;
    const int* x_rows;
    const int* tile_expert;
    const int* tile_row0;
    const int* num_tiles;
    const int* offsets;
    void* out;
    int* status;              // 0, or the code of the wait that gave up
    int F, K;
    int groups_per_tile;      // items of sixteen weight rows per tile: F / 8 for a pair, else F / 16
    int groups_per_expert;    // from one expert's first item to the next expert's, in the map's last coordinate
    int pieces;               // pieces of 64 k per stage
    int stages;
    int lists_final;          // the lists of tiles were complete before the kernel before this one began
};

template <int NB, bool PAIRED, typename OutT>
__global__ void __launch_bounds__(WS_THREADS, 1)
weight_stream_kernel(const __grid_constant__ CUtensorMap map_w, StreamParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[WS_MAX_STAGES], empty_bar[WS_MAX_STAGES];
    __shared__ int failed_flag;
    volatile int* failed = &failed_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t stage_bytes = (uint32_t)p.pieces * WS_PIECE_BYTES;
    float* reduce = reinterpret_cast<float*>(ring + (size_t)p.stages * stage_bytes);   // [2][warps][NB * 4][32]
    const int stage_k = p.pieces * WS_PIECE_K;
    const int stages_per_item = (p.K + stage_k - 1) / stage_k;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int s = 0; s < p.stages; ++s) { bar_init(&full_bar[s], 1); bar_init(&empty_bar[s], WS_COMPUTE_WARPS); }
        failed_flag = 0;
        bar_init_fence();
    }
    __syncthreads();

    if (warp == WS_COMPUTE_WARPS) {
        if (lane == 0) {
            bool waited = false;
            if (!p.lists_final) { wait_for_previous_kernel(); let_next_kernel_start(); waited = true; }
            const long long total = (long long)p.num_tiles[0] * p.groups_per_tile;
            const int begin = (int)(total * blockIdx.x / gridDim.x), end = (int)(total * (blockIdx.x + 1) / gridDim.x);
            // A step reads every weight once, so the lines of this stream are the first that L2 gives up again
            // (measured in a decode step of 16 layers: 1.79 -> 1.74 ms at batch 1, 5.06 -> 4.98 ms at batch 8).
            uint64_t leave_first = 0;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(leave_first));
            int s = 0, issued = 0;                         // the ring's next stage; stages asked for so far
            uint32_t parity = 0;                           // of the phase in which the stage's earlier use was given back
            int tile = begin / p.groups_per_tile, group = begin - tile * p.groups_per_tile;
            int tile_known = -1, e = 0;
            bool ok = true;
            for (int item = begin; item < end && ok; ++item) {
                if (tile != tile_known) { e = p.tile_expert[tile]; tile_known = tile; }
                const int coordinate = e * p.groups_per_expert + group;
                for (int st = 0; st < stages_per_item; ++st) {
                    if (issued >= p.stages) {
                        // the ring is full: from here on the kernel before this one is not needed for the lists, but the
                        // kernel after this one may only begin once this block has waited itself (see common.cuh)
                        if (!waited) { wait_for_previous_kernel(); let_next_kernel_start(); waited = true; }
                        if (!bar_wait(&empty_bar[s], parity, failed)) { atomicExch(p.status, 21); ok = false; break; }
                    }
                    bar_expect(&full_bar[s], stage_bytes);
                    load_5d_hint(ring + (size_t)s * stage_bytes, &map_w, 0, 0, 0, st * p.pieces, coordinate, &full_bar[s], leave_first);
                    ++issued;
                    if (++s == p.stages) { s = 0; if (issued > p.stages) parity ^= 1; }
                }
                if (++group == p.groups_per_tile) { group = 0; ++tile; }
            }
            if (!waited) { wait_for_previous_kernel(); let_next_kernel_start(); }
            if (*failed) {
                // copies may still be on their way into this block's shared memory: give each a bounded time to land
                // (a stage that was asked for u times before completes its phase u, whose parity is u & 1)
                for (int back = 0; back < p.stages && back < issued; ++back) {
                    const int q = issued - 1 - back;
                    int again = 0;
                    bar_wait(&full_bar[q % p.stages], (uint32_t)((q / p.stages) & 1), &again);
                }
            }
        }
    } else {
        wait_for_previous_kernel();
        let_next_kernel_start();
        const int g = lane >> 2, t = lane & 3;
        const int weight_row = (g >> 1) + 4 * (g & 1);                       // of its run of eight, for operand row g
        const long long total = (long long)p.num_tiles[0] * p.groups_per_tile;
        const int begin = (int)(total * blockIdx.x / gridDim.x), end = (int)(total * (blockIdx.x + 1) / gridDim.x);

        int s = 0, buffer = 0;
        uint32_t parity = 0;
        int tile = begin / p.groups_per_tile, group = begin - tile * p.groups_per_tile;
        int tile_known = -1, row0 = 0, rows = 1, blocks = 1;
        const bf16* xr[NB];
        bool ok = true;
        // this thread's 16 bytes of a row: chunk 4 half + t of the row's eight, swizzled with the row's number
        const uint32_t row_offset = warp * WS_PIECE_BYTES + weight_row * 128;
        const uint32_t chunk[2] = {(uint32_t)((t ^ weight_row) * 16), (uint32_t)(((4 + t) ^ weight_row) * 16)};
        for (int item = begin; item < end; ++item) {
            if (tile != tile_known) {
                tile_known = tile;
                row0 = p.tile_row0[tile];
                rows = min(NB * 8, p.offsets[p.tile_expert[tile] + 1] - row0);
                blocks = (rows + 7) >> 3;
#pragma unroll
                for (int j = 0; j < NB; ++j) {
                    const int r = min(j * 8 + g, rows - 1);                // rows past the end repeat the last one
                    const int src = p.x_rows ? p.x_rows[row0 + r] : row0 + r;
                    xr[j] = p.X + (size_t)src * p.K + 8 * t;
                }
            }
            float acc[NB][4];
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

            for (int st = 0; st < stages_per_item; ++st) {
                // the rows of x (from L1 mostly) are asked for before the wait for the weights
                uint4 xv[WS_PER_WARP][2][NB];
#pragma unroll
                for (int i = 0; i < WS_PER_WARP; ++i) {
                    const int k = st * stage_k + WS_PIECE_K * (warp + WS_COMPUTE_WARPS * i);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (warp + WS_COMPUTE_WARPS * i < p.pieces && k + 32 * half < p.K) {
#pragma unroll
                            for (int j = 0; j < NB; ++j)
                                if (j < blocks) xv[i][half][j] = __ldg(reinterpret_cast<const uint4*>(xr[j] + k + 32 * half));
                        }
                    }
                }
                int arrived = 1;
                if (lane == 0) arrived = bar_wait(&full_bar[s], parity, failed) ? 1 : 0;
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (!arrived) {
                    if (ok && lane == 0) atomicExch(p.status, 22);
                    ok = false;
                }
                const uint8_t* mine = ring + (size_t)s * stage_bytes + row_offset;
#pragma unroll
                for (int i = 0; i < WS_PER_WARP; ++i) {
                    const int k = st * stage_k + WS_PIECE_K * (warp + WS_COMPUTE_WARPS * i);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (warp + WS_COMPUTE_WARPS * i < p.pieces && k + 32 * half < p.K) {
                            const uint8_t* piece = mine + i * (WS_COMPUTE_WARPS * WS_PIECE_BYTES);
                            const uint4 lo = *reinterpret_cast<const uint4*>(piece + chunk[half]);            // first run of eight rows
                            const uint4 hi = *reinterpret_cast<const uint4*>(piece + 1024 + chunk[half]);     // second run
#pragma unroll
                            for (int j = 0; j < NB; ++j) {
                                if (j < blocks) {
                                    stream_mma(acc[j], lo.x, hi.x, lo.y, hi.y, xv[i][half][j].x, xv[i][half][j].y);
                                    stream_mma(acc[j], lo.z, hi.z, lo.w, hi.w, xv[i][half][j].z, xv[i][half][j].w);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) bar_arrive(&empty_bar[s]);
                if (++s == p.stages) { s = 0; parity ^= 1; }
            }

            // The warps' shares of the inner size are added in the order of the warps, by a warp that changes from
            // item to item, so that the sums and the stores delay no warp more than the others.
            float* shares = reduce + (size_t)buffer * WS_COMPUTE_WARPS * NB * 4 * 32;
            buffer ^= 1;
            const int adder = item % WS_COMPUTE_WARPS;
            if (warp != adder) {
#pragma unroll
                for (int j = 0; j < NB; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) shares[(warp * NB * 4 + j * 4 + i) * 32 + lane] = acc[j][i];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * WS_COMPUTE_WARPS) : "memory");
            if (warp == adder) {
                float sum[NB][4];
#pragma unroll
                for (int j = 0; j < NB; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sum[j][i] = adder == 0 ? acc[j][i] : shares[(j * 4 + i) * 32 + lane];
                for (int w = 1; w < WS_COMPUTE_WARPS; ++w)
#pragma unroll
                    for (int j = 0; j < NB; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) sum[j][i] += w == adder ? acc[j][i] : shares[(w * NB * 4 + j * 4 + i) * 32 + lane];
                if (ok && !*failed) {
                    OutT* out = (OutT*)p.out;
                    // accumulator i: the operand's row g + 8 (i >> 1), row 8 j + 2 t + (i & 1) of the tile
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
#pragma unroll
                        for (int i = 0; i < (PAIRED ? 2 : 4); ++i) {
                            const int r = j * 8 + 2 * t + (i & 1);
                            if (r >= rows) continue;
                            if (PAIRED) {
                                const float gate = sum[j][i], up = sum[j][i + 2];
                                out[(size_t)(row0 + r) * p.F + group * 8 + weight_row] = from_f32<OutT>(gate / (1.0f + expf(-gate)) * up);
                            } else {
                                out[(size_t)(row0 + r) * p.F + group * 16 + weight_row + 8 * (i >> 1)] = from_f32<OutT>(sum[j][i]);
                            }
                        }
                    }
                }
            }
            if (++group == p.groups_per_tile) { group = 0; ++tile; }
        }
    }
}

// W bf16 [E][(paired ? 2 : 1) F][K]; X bf16 rows of K; tiles of at most tile_rows (8, 16 or 32) rows.
// paired: out bf16 [N, F] = silu(x W1^T) * (x W3^T); else out float32 [N, F] = x W^T.
// lists_final: the lists of tiles do not depend on the kernel before this one in the stream.
// blocks: the most blocks to start; ring_kb: shared memory for the ring of stages; pieces: the most pieces of
// 64 k per stage (0: sixteen).
FRB_API int frb_weight_stream(const void* W, int num_experts, const void* X, const int* x_rows, const int* tile_expert,
                              const int* tile_row0, const int* num_tiles, const int* offsets, int max_tiles, int tile_rows,
                              void* out, int F, int K, int paired, int lists_final, int blocks, int ring_kb, int pieces, int* status,
                              cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    FRB_CHECK_ARG(K % WS_PIECE_K == 0 && K > 0, "weight stream: inner size %d is not a multiple of 64", K);
    FRB_CHECK_ARG(F > 0 && F % (paired ? 8 : 16) == 0, "weight stream: %d features are not a multiple of %d", F, paired ? 8 : 16);
    FRB_CHECK_ARG(tile_rows == 8 || tile_rows == 16 || tile_rows == 32, "weight stream: tiles of %d rows", tile_rows);
    FRB_CHECK_ARG(((uintptr_t)W & 15) == 0 && ((uintptr_t)X & 15) == 0, "weight stream: operands must be 16-byte aligned");
    FRB_CHECK_ARG(blocks > 0 && ring_kb >= 16 && ring_kb <= 200, "weight stream: %d blocks with a ring of %d KB", blocks, ring_kb);
    StreamParams p;
    p.X = (const bf16*)X; p.x_rows = x_rows; p.tile_expert = tile_expert; p.tile_row0 = tile_row0; p.num_tiles = num_tiles;
    p.offsets = offsets; p.out = out; p.status = status; p.F = F; p.K = K; p.lists_final = lists_final;
    p.groups_per_tile = paired ? F / 8 : F / 16;
    p.groups_per_expert = paired ? 2 * F / 8 : F / 16;
    // pieces per stage: as many as divide the inner size evenly, so that no stage is half empty; sixteen if none does
    const int all_pieces = K / WS_PIECE_K, most = pieces > 0 && pieces < WS_MAX_PIECES ? pieces : WS_MAX_PIECES;
    p.pieces = all_pieces <= most ? all_pieces : most;
    for (int c = most; c > most / 2 && all_pieces > most; --c)
        if (all_pieces % c == 0) { p.pieces = c; break; }
    const size_t stage_bytes = (size_t)p.pieces * WS_PIECE_BYTES;
    p.stages = (int)((size_t)ring_kb * 1024 / stage_bytes);
    if (p.stages > WS_MAX_STAGES) p.stages = WS_MAX_STAGES;
    if (p.stages < 2) p.stages = 2;
    CUtensorMap map_w;
    const uint64_t half_stride = paired ? (uint64_t)F * K : (uint64_t)8 * K;
    const uint64_t group_stride = paired ? (uint64_t)8 * K : (uint64_t)16 * K;
    const uint64_t groups = (uint64_t)(num_experts - 1) * p.groups_per_expert + p.groups_per_tile;
    FRB_CHECK_ARG(groups < (1ull << 31), "weight stream: %d experts of %d features exceed the tensor map", num_experts, F);
    FRB_CHECK_ARG(map_rows_in_pieces(&map_w, W, (uint64_t)K, half_stride, group_stride, groups, (uint32_t)p.pieces),
                  "weight stream: cuTensorMapEncodeTiled failed or is not available");
    const int nb = tile_rows / 8;
    const size_t beside_ring = (size_t)2 * WS_COMPUTE_WARPS * nb * 4 * 32 * sizeof(float) + 1024;
    while (p.stages > 2 && (size_t)p.stages * stage_bytes + beside_ring > 226 * 1024) --p.stages;   // what a block may have
    const size_t smem = (size_t)p.stages * stage_bytes + beside_ring;
    FRB_CHECK_ARG(smem <= 226 * 1024, "weight stream: two stages of %zu bytes do not fit a block's shared memory", stage_bytes);
    const long long items = (long long)max_tiles * p.groups_per_tile;
    FRB_CHECK_ARG(items < (1ll << 31), "weight stream: %d tiles of %d features exceed the launch", max_tiles, F);
    dim3 grid((unsigned)(items < blocks ? items : blocks));
#define LAUNCH(NB)                                                                                                          \
    if (paired) {                                                                                                           \
        cudaFuncSetAttribute(weight_stream_kernel<NB, true, bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        launch_dependent(weight_stream_kernel<NB, true, bf16>, grid, dim3(WS_THREADS), smem, stream, map_w, p);             \
    } else {                                                                                                                \
        cudaFuncSetAttribute(weight_stream_kernel<NB, false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_dependent(weight_stream_kernel<NB, false, float>, grid, dim3(WS_THREADS), smem, stream, map_w, p);           \
    }
    if (tile_rows == 8) { LAUNCH(1) } else if (tile_rows == 16) { LAUNCH(2) } else { LAUNCH(4) }
#undef LAUNCH
    FRB_RETURN_LAUNCH("weight_stream");
}
