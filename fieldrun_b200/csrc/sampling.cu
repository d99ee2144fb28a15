// Picking the next token of each row of float32 logits: the largest logit, or a sample of
// softmax(logits / temperature) by inverse CDF with one uniform number per row.
//
// The reference is greedy only: the largest logit, and on an exact tie the last index, as Rust's
// max_by returns (src/minimax.rs:375).  Temperature sampling has no counterpart there; the uniform
// numbers come from the host so that a plain implementation can repeat the choice.
#include "common.cuh"

#define SAMPLE_BLOCK 1024

__device__ __forceinline__ void keep_larger(float& best, int& best_i, float v, int i) {
    if (v > best || (v == best && i > best_i)) { best = v; best_i = i; }
}

// One block per row.  Each warp owns a contiguous range of the vocabulary, its lanes stride through it.
__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_rows_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, int* __restrict__ out) {
    after_previous_kernel();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float s_sum[32];
    __shared__ float s_max;
    __shared__ int s_pick;
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = logits + (size_t)row * vocab;
    const int per_warp = (((vocab + 31) / 32) + 31) / 32 * 32;        // multiple of 32 so ranges stay aligned
    const int begin = warp * per_warp, end = min(vocab, begin + per_warp);

    float best = -INFINITY;
    int best_i = -1;
    for (int i = begin + lane; i < end; i += 32) keep_larger(best, best_i, x[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        keep_larger(best, best_i, ov, oi);
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = -INFINITY;
        int bi = -1;
        for (int w = 0; w < 32; ++w) keep_larger(b, bi, s_val[w], s_idx[w]);
        s_max = b;
        s_pick = bi < 0 ? 0 : bi;
    }
    __syncthreads();
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {
        if (threadIdx.x == 0) out[row] = s_pick;
        return;
    }
    const float top = s_max, inv_t = 1.0f / temp;
    float part = 0.f;
    for (int i = begin + lane; i < end; i += 32) part += expf((x[i] - top) * inv_t);
    part = warp_sum(part);
    if (lane == 0) s_sum[warp] = part;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < 32; ++w) total += s_sum[w];
    const float target = uniform[row] * total;
    // the warp whose range holds the target
    float before = 0.f;
    int owner = -1;
    for (int w = 0; w < 32; ++w) {
        if (owner < 0 && before + s_sum[w] > target) owner = w;
        if (owner < 0) before += s_sum[w];
    }
    float scan_target = target;
    if (owner < 0) {            // rounding left the target at or past the total: the last token with weight
        owner = 31;
        while (owner > 0 && !(s_sum[owner] > 0.f)) --owner;
        scan_target = INFINITY;  // nothing crosses, so the range's last element with weight is taken below
    }
    if (warp != owner) return;
    float run = before;
    int pick = -1, last_positive = -1;
    for (int base = begin; base < end && pick < 0; base += 32) {
        const int i = base + lane;
        const float p = i < end ? expf((x[i] - top) * inv_t) : 0.f;
        float inc = p;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += up;
        }
        const unsigned crossed = __ballot_sync(0xffffffffu, i < end && run + inc > scan_target);
        const unsigned positive = __ballot_sync(0xffffffffu, p > 0.f);
        if (positive) last_positive = base + 31 - __clz(positive);
        if (crossed) pick = base + __ffs(crossed) - 1;
        run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (pick < 0) pick = last_positive >= 0 ? last_positive : s_pick;
    if (lane == 0) out[row] = pick;
}

// logits [rows, vocab] float32; temperature [rows] (null or <= 0: greedy); uniform [rows] in [0, 1).
FRB_API int frb_sample_rows(const float* logits, int rows, int vocab, const float* temperature, const float* uniform,
                            int* out, cudaStream_t stream) {
    if (rows == 0) return 0;
    FRB_CHECK_ARG(vocab >= 1, "sampling: a vocabulary of %d", vocab);
    FRB_CHECK_ARG(temperature == nullptr || uniform != nullptr, "sampling: temperatures without uniform numbers");
    launch_dependent(sample_rows_kernel, dim3(rows), dim3(SAMPLE_BLOCK), 0, stream, logits, vocab, temperature, uniform, out);
    FRB_RETURN_LAUNCH("sample_rows");
}
