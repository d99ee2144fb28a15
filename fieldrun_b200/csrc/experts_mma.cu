// Expert products for bfloat16 models as a stream over the experts' weights.
//
// y[row, f] = sum_k x[row, k] W_e[f, k] for the rows routed to expert e (src/minimax.rs:116-120).  A step
// has few rows per expert (one or two when decoding), so the weights are the traffic: every weight row is
// read once, straight from global memory into mma.sync fragments, and multiplied with all rows of the tile.
// The weights are the 16-row operand (16 output features per warp), the rows of x the 8-column operand;
// each thread loads 16 bytes (8 neighbouring k) per row for two MMAs -- the same regrouping of k on both
// operands, which a sum over k does not notice.  Accumulation is float32, in the same order for every
// row whatever else is in the batch.
//
// PAIRED: W = [E][2F][K] (gate rows then up rows); the epilogue writes silu(gate) * up as bfloat16.
// Otherwise W = [E][F][K] and the float32 products are written.
#include "common.cuh"

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// weights are read once: keep them out of L1, where the rows of x live
__device__ __forceinline__ uint4 load_stream(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

#define EM_MAX_GROUPS 4      // groups of 16 features per block: 1, 2 or 4; a block has groups * splits warps

// grid (row tile, block of 64 features).  NB column blocks of 8 rows each: the tile has at most 8 NB rows.
// The block's warps are (feature group, k split): with few tiles (a batch of one, or a dense layer as a
// single "expert") a block takes fewer feature groups and the inner dimension is cut into parts, so that
// there are enough blocks for every SM and enough loads in flight; the parts are added in the order of k,
// by the warps of the first part, through shared memory.
template <int NB, bool PAIRED, typename OutT>
__global__ void __launch_bounds__(512 / NB)
expert_gemm_mma_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, const int* __restrict__ x_rows,
                       const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                       const int* __restrict__ num_tiles, const int* __restrict__ offsets, OutT* __restrict__ out, int F, int K,
                       int k_per_split, int groups) {
    after_previous_kernel();
    extern __shared__ float partial[];       // [splits - 1][groups][NACC][32]
    constexpr int NACC = NB * 4 * (PAIRED ? 2 : 1);
    const int tile = blockIdx.x;
    if (tile >= num_tiles[0]) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int group = warp % groups, split = warp / groups, splits = blockDim.x / (32 * groups);
    const int f0 = (blockIdx.y * groups + group) * 16;
    const bool active = f0 < F;
    const int e = tile_expert[tile];
    const int row0 = tile_row0[tile];
    const int rows = min(NB * 8, offsets[e + 1] - row0);
    const int blocks = (rows + 7) >> 3;
    const size_t f_total = PAIRED ? (size_t)2 * F : (size_t)F;
    const bf16* wg0 = W + ((size_t)e * f_total + (active ? f0 : 0) + g) * K + 8 * t;      // feature f0 + g
    const bf16* wg1 = wg0 + (size_t)8 * K;                                 // feature f0 + g + 8
    const bf16* wu0 = wg0 + (size_t)F * K;                                 // the up rows of the same features
    const bf16* wu1 = wg1 + (size_t)F * K;
    const bf16* xr[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int r = min(j * 8 + g, rows - 1);                            // rows past the end repeat the last one
        const int src = x_rows ? x_rows[row0 + r] : row0 + r;
        xr[j] = X + (size_t)src * K + 8 * t;
    }
    float acc_g[NB][4], acc_u[PAIRED ? NB : 1][4];
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc_g[j][i] = 0.f; if (PAIRED) acc_u[j][i] = 0.f; }

    constexpr int UNROLL = NB == 1 ? 4 : 2;
    const int k_begin = split * k_per_split;
    const int k_end = active ? min(K, k_begin + k_per_split) : k_begin;
#pragma unroll 1
    for (int k0 = k_begin; k0 < k_end; k0 += 32 * UNROLL) {
        uint4 a_g0[UNROLL], a_g1[UNROLL], a_u0[PAIRED ? UNROLL : 1], a_u1[PAIRED ? UNROLL : 1];
#pragma unroll
        for (int s = 0; s < UNROLL; ++s) {
            if (k0 + 32 * s < k_end) {
                a_g0[s] = load_stream(wg0 + k0 + 32 * s);
                a_g1[s] = load_stream(wg1 + k0 + 32 * s);
                if (PAIRED) { a_u0[s] = load_stream(wu0 + k0 + 32 * s); a_u1[s] = load_stream(wu1 + k0 + 32 * s); }
            }
        }
#pragma unroll
        for (int s = 0; s < UNROLL; ++s) {
            if (k0 + 32 * s < k_end) {
#pragma unroll
                for (int j = 0; j < NB; ++j) {
                    if (j < blocks) {
                        const uint4 b = __ldg(reinterpret_cast<const uint4*>(xr[j] + k0 + 32 * s));
                        mma_bf16_16816(acc_g[j], a_g0[s].x, a_g1[s].x, a_g0[s].y, a_g1[s].y, b.x, b.y);
                        mma_bf16_16816(acc_g[j], a_g0[s].z, a_g1[s].z, a_g0[s].w, a_g1[s].w, b.z, b.w);
                        if (PAIRED) {
                            mma_bf16_16816(acc_u[j], a_u0[s].x, a_u1[s].x, a_u0[s].y, a_u1[s].y, b.x, b.y);
                            mma_bf16_16816(acc_u[j], a_u0[s].z, a_u1[s].z, a_u0[s].w, a_u1[s].w, b.z, b.w);
                        }
                    }
                }
            }
        }
    }
    if (splits > 1) {
        if (split > 0) {
            float* mine = partial + ((size_t)(split - 1) * groups + group) * NACC * 32 + lane;
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    mine[(j * 4 + i) * 32] = acc_g[j][i];
                    if (PAIRED) mine[(NB * 4 + j * 4 + i) * 32] = acc_u[j][i];
                }
        }
        __syncthreads();
        if (split > 0) return;
        for (int s = 1; s < splits; ++s) {
            const float* theirs = partial + ((size_t)(s - 1) * groups + group) * NACC * 32 + lane;
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc_g[j][i] += theirs[(j * 4 + i) * 32];
                    if (PAIRED) acc_u[j][i] += theirs[(NB * 4 + j * 4 + i) * 32];
                }
        }
    }
    if (!active) return;
    // accumulator (i): feature f0 + g + 8 (i >> 1), row 8 j + 2 t + (i & 1)
#pragma unroll
    for (int j = 0; j < NB; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = j * 8 + 2 * t + (i & 1);
            if (r >= rows) continue;
            const int f = f0 + g + 8 * (i >> 1);
            float v = acc_g[j][i];
            if (PAIRED) v = v / (1.0f + expf(-v)) * acc_u[j][i];
            out[(size_t)(row0 + r) * F + f] = from_f32<OutT>(v);
        }
    }
}

// W bf16 [E][(paired ? 2 : 1) F][K]; X bf16 rows of K; tiles of at most tile_rows (8, 16 or 32) rows.
// paired: out bf16 [N, F] = silu(x W1^T) * (x W3^T); else out float32 [N, F] = x W^T.
// splits: parts the inner size is cut into within a block (1 when there are many tiles); groups: groups of
// 16 features a block takes (4 when there are many tiles).
FRB_API int frb_expert_gemm_mma(const void* W, const void* X, const int* x_rows, const int* tile_expert, const int* tile_row0,
                                const int* num_tiles, const int* offsets, int max_tiles, int tile_rows, void* out, int F, int K,
                                int paired, int splits, int groups, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    FRB_CHECK_ARG(K % 32 == 0 && K > 0, "expert stream: inner size %d is not a multiple of 32", K);
    FRB_CHECK_ARG(F % 16 == 0 && F > 0, "expert stream: %d features are not a multiple of 16", F);
    FRB_CHECK_ARG(tile_rows == 8 || tile_rows == 16 || tile_rows == 32, "expert stream: tiles of %d rows", tile_rows);
    const int nb = tile_rows / 8;
    FRB_CHECK_ARG(groups == 1 || groups == 2 || groups == 4, "expert stream: %d feature groups per block", groups);
    FRB_CHECK_ARG(splits >= 1 && splits * groups * nb <= 16, "expert stream: %d splits x %d groups with tiles of %d rows exceed a block",
                  splits, groups, tile_rows);
    const int k_per_split = ((K + splits - 1) / splits + 127) / 128 * 128;
    dim3 grid(max_tiles, (F + 16 * groups - 1) / (16 * groups));
    FRB_CHECK_ARG(grid.y <= 65535, "expert stream: %d features exceed the grid", F);
    const int threads = 32 * groups * splits;
    const size_t smem = (size_t)(splits - 1) * groups * nb * 4 * (paired ? 2 : 1) * 32 * sizeof(float);
#define LAUNCH(NB)                                                                                                        \
    if (paired)                                                                                                           \
        launch_dependent(expert_gemm_mma_kernel<NB, true, bf16>, dim3(grid), dim3(threads), smem, stream,                                           \
            (const bf16*)W, (const bf16*)X, x_rows, tile_expert, tile_row0, num_tiles, offsets, (bf16*)out, F, K, k_per_split, groups); \
    else                                                                                                                  \
        launch_dependent(expert_gemm_mma_kernel<NB, false, float>, dim3(grid), dim3(threads), smem, stream,                                         \
            (const bf16*)W, (const bf16*)X, x_rows, tile_expert, tile_row0, num_tiles, offsets, (float*)out, F, K, k_per_split, groups)
    if (tile_rows == 8) { LAUNCH(1); } else if (tile_rows == 16) { LAUNCH(2); } else { LAUNCH(4); }
#undef LAUNCH
    FRB_RETURN_LAUNCH("expert_gemm_mma");
}
