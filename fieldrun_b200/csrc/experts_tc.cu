// Expert products on the fifth-generation tensor cores (tcgen05), for steps that bring many rows per
// expert (prompts).  Same formulas as the streamed kernel: PAIRED h = silu(x W1^T) * (x W3^T) from
// W = [E][2F][K], otherwise y = x W^T from W = [E][F][K]  (src/minimax.rs:116-120).
//
// One block computes 128 output features x NT rows of one expert: the weights are the 128-row operand of
// tcgen05.mma (they fill the tensor core's M whatever the number of rows), the rows of x its N <= 256.
// A producer thread moves [128 x 64] weight tiles and [NT x 64] row tiles into a ring of shared-memory
// stages with TMA (128-byte swizzle); one thread issues the MMAs, whose float32 accumulators live in
// tensor memory; four warps read them back with tcgen05.ld, apply the gate, and store.  With prompts of a
// few thousand tokens an expert sees a few dozen rows, so the step is bound by reading every weight once;
// the ring keeps well over a hundred KB of loads in flight per SM.
//
// Every wait on an mbarrier gives up after about a second, records a code in `status` and lets
// the block leave through the common exit, which frees the tensor memory; the host checks `status`.
#include "tcgen05.cuh"

#define TC_FEATS 128          // features per block: M of the MMA
#define TC_KBLOCK 64          // k per stage: 64 bf16 = one 128-byte swizzle row
#define TC_THREADS 192        // warp 0: TMA producer, warp 1: MMA issuer and tensor-memory owner, warps 2-5: epilogue

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

template <bool PAIRED, typename OutT>
__global__ void __launch_bounds__(TC_THREADS)
expert_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[8], empty_bar[8], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    // blocks that follow one another take the feature blocks of one tile: they read the same rows (which stay
    // in L2) and, where an expert has several tiles, the blocks of its next tile read the same weights soon after
    const int feature_blocks = p.F / TC_FEATS;
    const int tile = blockIdx.x / feature_blocks;
    if (tile >= p.num_tiles[0]) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = p.tile_expert[tile];
    const int row0 = p.tile_row0[tile];
    const int rows = min(p.NT, p.offsets[e + 1] - row0);
    const int f0 = (blockIdx.x - tile * feature_blocks) * TC_FEATS;
    const int f_total = PAIRED ? 2 * p.F : p.F;
    const int w_row_gate = e * f_total + f0, w_row_up = w_row_gate + p.F;
    const int k_blocks = p.K / TC_KBLOCK;
    const uint32_t w_bytes = TC_FEATS * TC_KBLOCK * 2, x_bytes = (uint32_t)p.NT * TC_KBLOCK * 2;
    const uint32_t stage_bytes = w_bytes * (PAIRED ? 2 : 1) + x_bytes;
    uint8_t* stage_base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);      // swizzled tiles: 1024-byte aligned

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { bar_init(&full_bar[s], 1); bar_init(&empty_bar[s], 1); }
        bar_init(&done_bar, 1);
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

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % p.stages;
                if (!bar_wait(&empty_bar[s], ((kb / p.stages) & 1) ^ 1, &failed)) { atomicExch(p.status, 1); break; }
                uint8_t* dst = stage_base + (size_t)s * stage_bytes;
                bar_expect(&full_bar[s], stage_bytes);
                load_2d(dst, &map_w, kb * TC_KBLOCK, w_row_gate, &full_bar[s]);
                if (PAIRED) load_2d(dst + w_bytes, &map_w, kb * TC_KBLOCK, w_row_up, &full_bar[s]);
                load_2d(dst + w_bytes * (PAIRED ? 2 : 1), &map_x, kb * TC_KBLOCK, row0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bf16 x bf16, both K-major, N = NT, M = 128
            const uint32_t idesc = instr_desc_bf16(TC_FEATS, p.NT);
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % p.stages;
                if (!bar_wait(&full_bar[s], (kb / p.stages) & 1, &failed)) { atomicExch(p.status, 2); ok = false; break; }
                fence_after_sync();
                const uint32_t base = smem_addr(stage_base + (size_t)s * stage_bytes);
                const uint32_t x_addr = base + w_bytes * (PAIRED ? 2 : 1);
#pragma unroll
                for (int k = 0; k < TC_KBLOCK / 16; ++k) {               // 16 k per MMA: 32 bytes along the swizzled row
                    const uint64_t desc_x = tile_desc(x_addr + k * 32);
                    mma_ss(tmem_base, tile_desc(base + k * 32), desc_x, idesc, (kb | k) != 0);
                    if (PAIRED) mma_ss(tmem_base + p.NT, tile_desc(base + w_bytes + k * 32), desc_x, idesc, (kb | k) != 0);
                }
                mma_commit(&empty_bar[s]);                              // the stage is free once these MMAs have read it
            }
            mma_commit(&done_bar);                                      // arrives when every MMA above has finished
        }
    } else {
        const int quarter = warp & 3;                                    // the 32 lanes of tensor memory this warp may read
        bool ok = bar_wait(&done_bar, 0, &failed);
        if (!ok && lane == 0) atomicExch(p.status, 3);
        fence_after_sync();
        if (ok && !failed) {
            const int f = f0 + quarter * 32 + lane;
            OutT* out = (OutT*)p.out;
            // 16 columns at a time, the next 16 on their way out of tensor memory while these are written
            const uint32_t lanes = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const int columns = min(p.NT, rows);
            uint32_t gate[2][16], up[2][16];
            tmem_ld16(lanes, gate[0]);
            if (PAIRED) tmem_ld16(lanes + p.NT, up[0]);
#pragma unroll 1
            for (int c0 = 0; c0 < columns; c0 += 32) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int c = c0 + 16 * half;
                    if (c >= columns) break;
                    tmem_wait_ld();
                    if (c + 16 < columns) {
                        tmem_ld16(lanes + c + 16, gate[half ^ 1]);
                        if (PAIRED) tmem_ld16(lanes + p.NT + c + 16, up[half ^ 1]);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int n = c + j;
                        if (n < rows) {
                            float v = __uint_as_float(gate[half][j]);
                            // silu(gate) * up; the result is rounded to bfloat16, so the fast exponential and division do
                            if (PAIRED) v = __fdividef(v, 1.0f + __expf(-v)) * __uint_as_float(up[half][j]);
                            out[(size_t)(row0 + n) * p.F + f] = from_f32<OutT>(v);
                        }
                    }
                }
            }
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
    const int cols = paired ? 2 * tile_rows : tile_rows;
    p.tmem_cols = cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
    const size_t stage_bytes = (size_t)TC_FEATS * TC_KBLOCK * 2 * (paired ? 2 : 1) + (size_t)tile_rows * TC_KBLOCK * 2;
    // Two blocks per SM when both the stages (at least two each) and the accumulators fit twice: one block's
    // set-up and epilogue then overlap the other's stream of weights.  Otherwise one block with a deeper ring.
    const bool two_per_sm = 2 * stage_bytes <= 110 * 1024 && p.tmem_cols <= 256;
    int stages = (int)(((two_per_sm ? 110 : 200) * 1024) / stage_bytes);
    p.stages = stages > 8 ? 8 : stages;
    const size_t smem = p.stages * stage_bytes + 1024;
    FRB_CHECK_ARG((long long)max_tiles * (F / TC_FEATS) < (1ll << 31), "expert tensor-core product: %d tiles of %d features exceed the grid",
                  max_tiles, F);
    dim3 grid((unsigned)max_tiles * (F / TC_FEATS));
    if (paired) {
        cudaFuncSetAttribute(expert_gemm_tc_kernel<true, bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        expert_gemm_tc_kernel<true, bf16><<<grid, TC_THREADS, smem, stream>>>(map_w, map_x, p);
    } else {
        cudaFuncSetAttribute(expert_gemm_tc_kernel<false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        expert_gemm_tc_kernel<false, float><<<grid, TC_THREADS, smem, stream>>>(map_w, map_x, p);
    }
    FRB_RETURN_LAUNCH("expert_gemm_tc");
}

// out[i, :] = x[rows[i], :]: the rows of a step put in expert-sorted order, so that a tile of an expert's
// rows is one box of a tensor map.
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ rows, uint4* __restrict__ out, int vec_per_row) {
    const int i = blockIdx.x;
    const uint4* src = x + (size_t)rows[i] * vec_per_row;
    uint4* dst = out + (size_t)i * vec_per_row;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = src[v];
}

FRB_API int frb_gather_rows_bf16(const void* x, const int* rows, void* out, int num_rows, int width, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(width % 8 == 0, "gather: a width of %d is not a multiple of 8", width);
    gather_rows_kernel<<<num_rows, 128, 0, stream>>>((const uint4*)x, rows, (uint4*)out, width / 8);
    FRB_RETURN_LAUNCH("gather_rows");
}
