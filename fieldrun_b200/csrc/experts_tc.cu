// Expert products on the fifth-generation tensor cores (tcgen05), for steps that bring many rows per
// expert (prompts).  Same formulas as the streamed kernel: PAIRED h = silu(x W1^T) * (x W3^T) from
// W = [E][2F][K], otherwise y = x W^T from W = [E][F][K]  (src/minimax.rs:116-120).
//
// An item of work is 128 output features x NT rows of one expert: the weights are the 128-row operand of
// tcgen05.mma (they fill the tensor core's M whatever the number of rows), the rows of x its N <= 256.
// Blocks stay for the whole launch (one or two per SM) and take items in turn.  A producer thread moves
// [128 x 64] weight tiles and [NT x 64] row tiles into a ring of shared-memory stages with TMA (128-byte
// swizzle), running ahead into the next item; one thread issues the MMAs, whose float32 accumulators live in
// tensor memory; four or eight warps read them back with tcgen05.ld, apply the gate, and store.  With prompts of a
// few thousand tokens an expert sees a few dozen rows, so the step is bound by reading every weight once;
// the ring keeps well over a hundred KB of loads in flight per SM.
//
// Every wait on an mbarrier gives up after about a second, records a code in `status` and lets
// the block leave through the common exit, which frees the tensor memory; the host checks `status`.
#include "tcgen05.cuh"

#define TC_FEATS 128          // features per block: M of the MMA
#define TC_KBLOCK 64          // k per stage: 64 bf16 = one 128-byte swizzle row
// warp 0: TMA producer, warp 1: MMA issuer and tensor-memory owner, then EW = 4 or 8 epilogue warps (8 where a block
// has the SM to itself: with 4, two blocks' registers fit an SM)
#define TC_THREADS(EW) (64 + 32 * (EW))

using namespace frb_tma;
using namespace frb_tc;

struct TcParams {
    const int* tile_expert;
    const int* tile_row0;
    const int* num_tiles;
    const int* offsets;
    void* out;
    int* status;             // 0, or the code of the wait that gave up
    int F, K, NT, stages, tmem_cols;
};

// WIDE (not PAIRED): the block takes 256 features, as two accumulators of 128 over the same rows: a stage then
// feeds twice the arithmetic from the same tile of rows, which matters where the tiles come out of L2 as fast as
// an SM can take them.
template <bool PAIRED, bool WIDE, int EW, typename OutT>
__global__ void __launch_bounds__(TC_THREADS(EW), EW == 4 ? 2 : 1)
expert_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    // done_bar: the accumulators of the block's current item are complete; read_bar: the epilogue has read them
    __shared__ uint64_t full_bar[8], empty_bar[8], done_bar, read_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    constexpr bool TWO = PAIRED || WIDE;                       // two accumulators, two tiles of weights a stage
    constexpr int BLOCK_FEATS = WIDE ? 2 * TC_FEATS : TC_FEATS;
    // A block stays for the whole launch and takes the items blockIdx.x, blockIdx.x + gridDim.x, ...: an item is a
    // feature block of a tile.  Items that follow one another are the feature blocks of one tile: the blocks that
    // run side by side read the same rows (which stay in L2) and, where an expert has several tiles, the same
    // weights soon after.  The ring of stages runs on from item to item, so the next item's first tiles arrive
    // while the epilogue still reads this item's accumulators.
    let_next_kernel_start();
    const int feature_blocks = p.F / BLOCK_FEATS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f_total = PAIRED ? 2 * p.F : p.F;
    const int k_blocks = p.K / TC_KBLOCK;
    const uint32_t w_bytes = TC_FEATS * TC_KBLOCK * 2, x_bytes = (uint32_t)p.NT * TC_KBLOCK * 2;
    const uint32_t stage_bytes = w_bytes * (TWO ? 2 : 1) + x_bytes;
    uint8_t* stage_base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);      // swizzled tiles: 1024-byte aligned

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { bar_init(&full_bar[s], 1); bar_init(&empty_bar[s], 1); }
        bar_init(&done_bar, 1);
        bar_init(&read_bar, EW);
        failed = 0;
        bar_init_fence();
    }
    if (warp == 1) {                                            // one warp allocates the accumulators' columns
        tmem_alloc(&tmem_base_slot, (uint32_t)p.tmem_cols);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    wait_for_previous_kernel();                                  // barriers and tensor memory were set up while it still ran
    const int num_items = p.num_tiles[0] * feature_blocks;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t parity = 1;                                 // of the phase in which the stage's earlier use was given back
            bool ok = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const int tile = item / feature_blocks;
                const int e = p.tile_expert[tile], row0 = p.tile_row0[tile];
                const int w_row_gate = e * f_total + (item - tile * feature_blocks) * BLOCK_FEATS;
                const int w_row_up = w_row_gate + (PAIRED ? p.F : TC_FEATS);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!bar_wait(&empty_bar[s], parity, &failed)) { atomicExch(p.status, 1); ok = false; break; }
                    uint8_t* dst = stage_base + (size_t)s * stage_bytes;
                    bar_expect(&full_bar[s], stage_bytes);
                    load_2d(dst, &map_w, kb * TC_KBLOCK, w_row_gate, &full_bar[s]);
                    if (TWO) load_2d(dst + w_bytes, &map_w, kb * TC_KBLOCK, w_row_up, &full_bar[s]);
                    load_2d(dst + w_bytes * (TWO ? 2 : 1), &map_x, kb * TC_KBLOCK, row0, &full_bar[s]);
                    if (++s == p.stages) { s = 0; parity ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bf16 x bf16, both K-major, N = NT, M = 128
            const uint32_t idesc = instr_desc_bf16(TC_FEATS, p.NT);
            int s = 0;
            uint32_t parity = 0, read_parity = 0;
            bool ok = true, first = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                if (!first) {                                    // the item before has left the accumulators
                    if (!bar_wait(&read_bar, read_parity, &failed)) { atomicExch(p.status, 6); ok = false; break; }
                    read_parity ^= 1;
                    fence_after_sync();
                }
                first = false;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!bar_wait(&full_bar[s], parity, &failed)) { atomicExch(p.status, 2); ok = false; break; }
                    fence_after_sync();
                    const uint32_t base = smem_addr(stage_base + (size_t)s * stage_bytes);
                    const uint32_t x_addr = base + w_bytes * (TWO ? 2 : 1);
#pragma unroll
                    for (int k = 0; k < TC_KBLOCK / 16; ++k) {           // 16 k per MMA: 32 bytes along the swizzled row
                        const uint64_t desc_x = tile_desc(x_addr + k * 32);
                        mma_ss(tmem_base, tile_desc(base + k * 32), desc_x, idesc, (kb | k) != 0);
                        if (TWO) mma_ss(tmem_base + p.NT, tile_desc(base + w_bytes + k * 32), desc_x, idesc, (kb | k) != 0);
                    }
                    mma_commit(&empty_bar[s]);                          // the stage is free once these MMAs have read it
                    if (++s == p.stages) { s = 0; parity ^= 1; }
                }
                if (ok) mma_commit(&done_bar);                          // arrives when every MMA above has finished
            }
        }
    } else {
        // Epilogue: warp w reads the 32 lanes of tensor memory that it may (w & 3); the two warps of a quarter take
        // the groups of 16 columns in turn.
        const int quarter = warp & 3, turn = (warp - 2) >> 2;
        const uint32_t lanes = tmem_base + ((uint32_t)(quarter * 32) << 16);
        OutT* out = (OutT*)p.out;
        uint32_t done_parity = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            const int tile = item / feature_blocks;
            const int e = p.tile_expert[tile], row0 = p.tile_row0[tile];
            const int rows = min(p.NT, p.offsets[e + 1] - row0);
            const int f = (item - tile * feature_blocks) * BLOCK_FEATS + quarter * 32 + lane;
            if (!bar_wait(&done_bar, done_parity, &failed)) { if (lane == 0) atomicExch(p.status, 3); ok = false; break; }
            done_parity ^= 1;
            fence_after_sync();
            // 16 columns at a time, the next 16 on their way out of tensor memory while these are written
            constexpr int STEP = 16 * (EW / 4);
            uint32_t gate[2][16], up[2][16];
            int c = 16 * turn;
            if (c < rows) {
                tmem_ld16(lanes + c, gate[0]);
                if (TWO) tmem_ld16(lanes + p.NT + c, up[0]);
            }
#pragma unroll 1
            for (; c < rows; c += 2 * STEP) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int c0 = c + STEP * half;
                    if (c0 >= rows) break;
                    tmem_wait_ld();
                    if (c0 + STEP < rows) {
                        tmem_ld16(lanes + c0 + STEP, gate[half ^ 1]);
                        if (TWO) tmem_ld16(lanes + p.NT + c0 + STEP, up[half ^ 1]);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int n = c0 + j;
                        if (n < rows) {
                            float v = __uint_as_float(gate[half][j]);
                            // silu(gate) * up; the result is rounded to bfloat16, so the fast exponential and division do
                            if (PAIRED) v = __fdividef(v, 1.0f + __expf(-v)) * __uint_as_float(up[half][j]);
                            out[(size_t)(row0 + n) * p.F + f] = from_f32<OutT>(v);
                            if (WIDE) out[(size_t)(row0 + n) * p.F + f + TC_FEATS] = from_f32<OutT>(__uint_as_float(up[half][j]));
                        }
                    }
                }
            }
            tmem_wait_ld();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) bar_arrive(&read_bar);                // this warp has what it needs of the accumulators
        }
    }
    fence_before_sync();
    __syncthreads();
    if (failed && warp == 0 && lane == 0) {
        // copies may still be on their way into this block's shared memory: give them a bounded time to land
        for (int s = 0; s < p.stages; ++s) { int again = 0; bar_wait(&full_bar[s], 0, &again); }
    }
    __syncthreads();
    if (warp == 1) {
        tmem_free(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// ----------------------------------------------------------------------------- host side

// W bf16 [E][(paired ? 2 : 1) F][K]; X bf16 [x_rows_total, K] with the rows of each expert together (sorted
// order); tiles of tile_rows = 32, 64, 128 or 256 rows.  status: one int on the device, zero before the call.
FRB_API int frb_expert_gemm_tc(const void* W, int num_experts, const void* X, int x_rows_total, const int* tile_expert,
                               const int* tile_row0, const int* num_tiles, const int* offsets, int max_tiles, int tile_rows,
                               void* out, int F, int K, int paired, int* status, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    FRB_CHECK_ARG(K % TC_KBLOCK == 0 && K > 0, "expert tensor-core product: inner size %d is not a multiple of 64", K);
    FRB_CHECK_ARG(F % TC_FEATS == 0 && F > 0, "expert tensor-core product: %d features are not a multiple of 128", F);
    FRB_CHECK_ARG(tile_rows == 32 || tile_rows == 64 || tile_rows == 128 || tile_rows == 256,
                  "expert tensor-core product: tiles of %d rows", tile_rows);
    FRB_CHECK_ARG(((uintptr_t)W & 15) == 0 && ((uintptr_t)X & 15) == 0, "expert tensor-core product: operands must be 16-byte aligned");
    CUtensorMap map_w, map_x;
    const uint64_t w_rows = (uint64_t)num_experts * (paired ? 2 : 1) * F;
    FRB_CHECK_ARG(map_rows_of_64(&map_w, W, w_rows, K, TC_FEATS) && map_rows_of_64(&map_x, X, x_rows_total, K, tile_rows),
                  "expert tensor-core product: cuTensorMapEncodeTiled failed or is not available");
    TcParams p;
    p.tile_expert = tile_expert; p.tile_row0 = tile_row0; p.num_tiles = num_tiles; p.offsets = offsets; p.out = out;
    p.status = status; p.F = F; p.K = K; p.NT = tile_rows;
    // products of one matrix take 256 features a block where the tiles are large and arithmetic is the bound
    const bool wide = !paired && tile_rows >= 128 && F % (2 * TC_FEATS) == 0;
    const bool two = paired || wide;
    const int cols = two ? 2 * tile_rows : tile_rows;
    p.tmem_cols = cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
    const size_t stage_bytes = (size_t)TC_FEATS * TC_KBLOCK * 2 * (two ? 2 : 1) + (size_t)tile_rows * TC_KBLOCK * 2;
    // Two blocks per SM when both the stages (at least two each) and the accumulators fit twice: one block's
    // set-up and epilogue then overlap the other's stream of weights.  Otherwise one block with a deeper ring.
    const bool two_per_sm = 2 * stage_bytes <= 110 * 1024 && p.tmem_cols <= 256;
    int stages = (int)(((two_per_sm ? 110 : 200) * 1024) / stage_bytes);
    p.stages = stages > 8 ? 8 : stages;
    const size_t smem = p.stages * stage_bytes + 1024;
    const long long most_items = (long long)max_tiles * (F / (wide ? 2 * TC_FEATS : TC_FEATS));
    FRB_CHECK_ARG(most_items < (1ll << 31), "expert tensor-core product: %d tiles of %d features exceed the count of items", max_tiles, F);
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long resident = (long long)sms * (two_per_sm ? 2 : 1);           // the blocks stay; each takes every resident-th item
    dim3 grid((unsigned)(most_items < resident ? most_items : resident));
#define FRB_TC_LAUNCH(PAIRED, WIDE, EW, OutT)                                                                              \
    do {                                                                                                                   \
        cudaFuncSetAttribute(expert_gemm_tc_kernel<PAIRED, WIDE, EW, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_dependent_resident(EW == 4 ? 2 : 1, expert_gemm_tc_kernel<PAIRED, WIDE, EW, OutT>, grid, dim3(TC_THREADS(EW)), smem, \
                                  stream, map_w, map_x, p);                                                                 \
    } while (0)
    if (paired) { if (two_per_sm) FRB_TC_LAUNCH(true, false, 4, bf16); else FRB_TC_LAUNCH(true, false, 8, bf16); }
    else if (wide) { if (two_per_sm) FRB_TC_LAUNCH(false, true, 4, float); else FRB_TC_LAUNCH(false, true, 8, float); }
    else { if (two_per_sm) FRB_TC_LAUNCH(false, false, 4, float); else FRB_TC_LAUNCH(false, false, 8, float); }
#undef FRB_TC_LAUNCH
    FRB_RETURN_LAUNCH("expert_gemm_tc");
}

// out[i, :] = x[rows[i], :]: the rows of a step put in expert-sorted order, so that a tile of an expert's
// rows is one box of a tensor map.
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ rows, uint4* __restrict__ out, int num_rows,
                                   int vec_per_row) {
    after_previous_kernel();
    for (int i = blockIdx.x; i < num_rows; i += gridDim.x) {
        const uint4* src = x + (size_t)rows[i] * vec_per_row;
        uint4* dst = out + (size_t)i * vec_per_row;
        for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = src[v];
    }
}

FRB_API int frb_gather_rows_bf16(const void* x, const int* rows, void* out, int num_rows, int width, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(width % 8 == 0, "gather: a width of %d is not a multiple of 8", width);
    // started early where a block has a row (a short prompt); many rows take every block several
    launch_dependent(gather_rows_kernel, dim3((unsigned)(num_rows < 65536 ? num_rows : 65536)), dim3(128), 0, stream, (const uint4*)x, rows,
                     (uint4*)out, num_rows, width / 8);
    FRB_RETURN_LAUNCH("gather_rows");
}
