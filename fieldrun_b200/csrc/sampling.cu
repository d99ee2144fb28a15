// Picking the next token of each row of float32 logits: the largest logit, or a sample of
// softmax(logits / temperature) by inverse CDF with one uniform number per row, optionally among the
// top_k largest logits and the smallest set of them that holds top_p of the probability.
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
                   const float* __restrict__ uniform, const float* __restrict__ floor, int* __restrict__ out) {
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
    const float least = floor ? floor[row] : -INFINITY;              // logits below it have no weight (top-k, top-p)
    float part = 0.f;
    for (int i = begin + lane; i < end; i += 32) part += x[i] >= least ? expf((x[i] - top) * inv_t) : 0.f;
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
        const float p = (i < end && x[i] >= least) ? expf((x[i] - top) * inv_t) : 0.f;
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

// logits [rows, vocab] float32; temperature [rows] (null or <= 0: greedy); uniform [rows] in [0, 1); floor [rows] or
// null: the smallest logit that may be picked (from frb_sample_floor).
FRB_API int frb_sample_rows(const float* logits, int rows, int vocab, const float* temperature, const float* uniform,
                            const float* floor, int* out, cudaStream_t stream) {
    if (rows == 0) return 0;
    FRB_CHECK_ARG(vocab >= 1, "sampling: a vocabulary of %d", vocab);
    FRB_CHECK_ARG(temperature == nullptr || uniform != nullptr, "sampling: temperatures without uniform numbers");
    launch_dependent(sample_rows_kernel, dim3(rows), dim3(SAMPLE_BLOCK), 0, stream, logits, vocab, temperature, uniform, floor, out);
    FRB_RETURN_LAUNCH("sample_rows");
}

// ----------------------------------------------------------------------------- top-k and top-p

// Floats as unsigned integers in the same order.
__device__ __forceinline__ unsigned int sample_key(float v) {
    const unsigned int u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float sample_unkey(unsigned int k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

#define SAMPLE_MASS_BITS 40      // a token's weight exp((x - max) / T) in (0, 1] is counted in units of 2^-40

// One block per row finds the smallest logit that stays: among the logits in descending order, the k-th
// (top_k > 0), or the one with which the weights exp((x - max) / T) first add up to top_p of their total
// (top_p < 1), whichever comes first; equal logits stay or go together.  It is a radix selection over the
// logits' bits, eight at a time from the top: a histogram of how many logits, and how much weight, fall
// into each of the 256 values of the next eight bits among those that share the bits found so far.  The
// weights are added as integers (units of 2^-40), so that the sums do not depend on the order of the adds.
// Neither has a counterpart in the reference, which is greedy only (src/minimax.rs:375).
__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_floor_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                    const int* __restrict__ top_k, const float* __restrict__ top_p, float* __restrict__ floor) {
    after_previous_kernel();
    __shared__ unsigned int s_count[256];
    __shared__ unsigned long long s_mass[256];
    __shared__ float s_red[32];
    __shared__ unsigned int s_prefix;
    __shared__ unsigned long long s_want_mass;
    __shared__ unsigned int s_want_count;
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = logits + (size_t)row * vocab;
    const float temp = temperature ? temperature[row] : 0.f;
    const int k = top_k ? top_k[row] : 0;
    const float p = top_p ? top_p[row] : 1.f;
    if (!(temp > 0.f) || (k <= 0 && !(p < 1.f))) {                    // greedy, or nothing to cut
        if (threadIdx.x == 0) floor[row] = -INFINITY;
        return;
    }
    float top = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += SAMPLE_BLOCK) top = fmaxf(top, x[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    if (lane == 0) s_red[warp] = top;
    __syncthreads();
    top = s_red[0];
    for (int w = 1; w < 32; ++w) top = fmaxf(top, s_red[w]);
    const float inv_t = 1.0f / temp;
    const float unit = (float)(1ull << SAMPLE_MASS_BITS);
    if (threadIdx.x == 0) {
        s_prefix = 0;
        s_want_count = k > 0 ? (unsigned int)k : 0xffffffffu;
        s_want_mass = 0;
    }
    for (int i = threadIdx.x; i < 256; i += SAMPLE_BLOCK) { s_count[i] = 0; s_mass[i] = 0; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
        const unsigned int prefix = s_prefix;
        const unsigned int above = shift == 24 ? 0u : 0xffffffffu << (shift + 8);      // the bits found so far
        for (int i = threadIdx.x; i < vocab; i += SAMPLE_BLOCK) {
            const unsigned int key = sample_key(x[i]);
            if ((key & above) == prefix) {
                const unsigned int digit = (key >> shift) & 255u;
                atomicAdd(&s_count[digit], 1u);
                atomicAdd(&s_mass[digit], (unsigned long long)(expf((x[i] - top) * inv_t) * unit));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            if (shift == 24) {                   // the first histogram holds every logit: the total weight
                unsigned long long all = 0;
                for (int d = 0; d < 256; ++d) all += s_mass[d];
                s_want_mass = p < 1.f ? (unsigned long long)((double)all * (double)p) : ~0ull;
            }
            unsigned int count = 0;
            unsigned long long mass = 0;
            int d = 255;
            for (; d > 0; --d) {                 // from the largest logits down: the value that holds the last one to stay
                if (count + s_count[d] >= s_want_count || (s_mass[d] > 0 && mass + s_mass[d] >= s_want_mass)) break;
                count += s_count[d];
                mass += s_mass[d];
            }
            s_prefix = prefix | ((unsigned int)d << shift);
            s_want_count = s_want_count == 0xffffffffu ? 0xffffffffu : s_want_count - count;
            s_want_mass = s_want_mass == ~0ull ? ~0ull : s_want_mass - mass;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 256; i += SAMPLE_BLOCK) { s_count[i] = 0; s_mass[i] = 0; }
        __syncthreads();
    }
    if (threadIdx.x == 0) floor[row] = sample_unkey(s_prefix);
}

// floor[row] = the smallest logit of the row that sampling may pick (see the kernel); -inf where the row is
// greedy or neither top_k (> 0) nor top_p (< 1) cuts anything.  top_k, top_p: [rows] or null.
FRB_API int frb_sample_floor(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                             const float* top_p, float* floor, cudaStream_t stream) {
    if (rows == 0) return 0;
    FRB_CHECK_ARG(vocab >= 1, "sampling: a vocabulary of %d", vocab);
    launch_dependent(sample_floor_kernel, dim3(rows), dim3(SAMPLE_BLOCK), 0, stream, logits, vocab, temperature, top_k, top_p, floor);
    FRB_RETURN_LAUNCH("sample_floor");
}
