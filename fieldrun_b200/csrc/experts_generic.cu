// Expert products over expert-sorted rows, any sizes, float32 accumulation in k order.
// It is the expert path of the float32 model and the fallback of the bfloat16 model for sizes the
// tensor-core kernels refuse.
//
// PAIRED: h = silu(x W1^T) * (x W3^T) with W = [E][2F][K] holding the F gate rows then the F up rows;
// otherwise y = x W^T with W = [E][F][K]  (src/minimax.rs:116-120; silu(x) = x/(1+exp(-x)), :31).
#include "common.cuh"

#define EG_ROWS 32
#define EG_FEATS 64
#define EG_K 16

template <typename T, typename OutT, bool PAIRED>
__global__ void __launch_bounds__(256)
expert_gemm_generic_kernel(const T* __restrict__ W, const T* __restrict__ X, const int* __restrict__ x_rows,
                           const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                           const int* __restrict__ num_tiles, const int* __restrict__ offsets, OutT* __restrict__ out,
                           int F, int K) {
    __shared__ float xs[EG_K][EG_ROWS + 1];
    __shared__ float wg[EG_K][EG_FEATS + 1];
    __shared__ float wu[PAIRED ? EG_K : 1][EG_FEATS + 1];
    const int tile = blockIdx.x;
    if (tile >= num_tiles[0]) return;
    const int e = tile_expert[tile];
    const int row0 = tile_row0[tile];
    const int rows = min(EG_ROWS, offsets[e + 1] - row0);
    const int f0 = blockIdx.y * EG_FEATS;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const size_t f_total = PAIRED ? (size_t)2 * F : (size_t)F;
    const T* We = W + (size_t)e * f_total * K;

    float acc_g[2][4], acc_u[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc_g[i][j] = 0.f; acc_u[i][j] = 0.f; }

    for (int k0 = 0; k0 < K; k0 += EG_K) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = tid + 256 * it, r = idx >> 4, kk = idx & 15;
            float v = 0.f;
            if (r < rows && k0 + kk < K) {
                const int src = x_rows ? x_rows[row0 + r] : row0 + r;
                v = to_f32<T>(X[(size_t)src * K + k0 + kk]);
            }
            xs[kk][r] = v;
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + 256 * it, f = idx >> 4, kk = idx & 15;
            const bool ok = (f0 + f < F) && (k0 + kk < K);
            wg[kk][f] = ok ? to_f32<T>(We[(size_t)(f0 + f) * K + k0 + kk]) : 0.f;
            if (PAIRED) wu[kk][f] = ok ? to_f32<T>(We[((size_t)F + f0 + f) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < EG_K; ++kk) {
            const float x0 = xs[kk][ty * 2], x1 = xs[kk][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float g = wg[kk][tx * 4 + j];
                acc_g[0][j] += x0 * g;
                acc_g[1][j] += x1 * g;
                if (PAIRED) {
                    const float u = wu[kk][tx * 4 + j];
                    acc_u[0][j] += x0 * u;
                    acc_u[1][j] += x1 * u;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = f0 + tx * 4 + j;
            if (f >= F) continue;
            float v = acc_g[i][j];
            if (PAIRED) v = v / (1.0f + expf(-v)) * acc_u[i][j];
            out[(size_t)(row0 + r) * F + f] = from_f32<OutT>(v);
        }
    }
}

// W [E][(paired ? 2 : 1) * F][K]; X rows of K; out [N, F].  x_rows (nullable) maps a sorted row to its X row.
// max_tiles bounds the grid; blocks beyond num_tiles[0] leave at once.
FRB_API int frb_expert_gemm_generic(const void* W, const void* X, int dtype, const int* x_rows, const int* tile_expert,
                                    const int* tile_row0, const int* num_tiles, const int* offsets, int max_tiles,
                                    void* out, int out_dtype, int F, int K, int paired, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    dim3 grid(max_tiles, (F + EG_FEATS - 1) / EG_FEATS);
    FRB_CHECK_ARG(grid.y <= 65535, "expert product: %d features exceed the grid", F);
#define LAUNCH(T, OutT, P)                                                                                              \
    expert_gemm_generic_kernel<T, OutT, P><<<grid, 256, 0, stream>>>((const T*)W, (const T*)X, x_rows, tile_expert,      \
                                                                     tile_row0, num_tiles, offsets, (OutT*)out, F, K)
    FRB_DISPATCH_DTYPE(dtype, T, FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        if (paired) LAUNCH(T, OutT, true); else LAUNCH(T, OutT, false);
    }));
#undef LAUNCH
    FRB_RETURN_LAUNCH("expert_gemm_generic");
}
