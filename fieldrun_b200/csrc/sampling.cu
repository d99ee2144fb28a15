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

// The largest logit of every row in two launches, for large vocabularies: one block scanning a row of 200,064 logits
// alone takes 15 us (what one SM can read), 32 blocks a row and a warp to pick among their results 4.
#define ARGMAX_SLICES 32
#define ARGMAX_BLOCK 256

// grid (slice, row): the largest logit of a slice of the row, the last index among equal ones
__global__ void __launch_bounds__(ARGMAX_BLOCK)
argmax_slices_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ slice_val, int* __restrict__ slice_idx) {
    after_previous_kernel();
    __shared__ float s_val[ARGMAX_BLOCK / 32];
    __shared__ int s_idx[ARGMAX_BLOCK / 32];
    const int slice = blockIdx.x, row = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = logits + (size_t)row * vocab;
    const int per_slice = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int begin = slice * per_slice, end = min(vocab, begin + per_slice);
    float best = -INFINITY;
    int best_i = -1;
    constexpr int AT_ONCE = 8;                                          // loads on their way at a time
    int i = begin + threadIdx.x;
    for (; i + (AT_ONCE - 1) * ARGMAX_BLOCK < end; i += AT_ONCE * ARGMAX_BLOCK) {
        float v[AT_ONCE];
#pragma unroll
        for (int u = 0; u < AT_ONCE; ++u) v[u] = x[i + u * ARGMAX_BLOCK];
#pragma unroll
        for (int u = 0; u < AT_ONCE; ++u) keep_larger(best, best_i, v[u], i + u * ARGMAX_BLOCK);
    }
    for (; i < end; i += ARGMAX_BLOCK) keep_larger(best, best_i, x[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        keep_larger(best, best_i, ov, oi);
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < ARGMAX_BLOCK / 32; ++w) keep_larger(best, best_i, s_val[w], s_idx[w]);
        slice_val[row * ARGMAX_SLICES + slice] = best;
        slice_idx[row * ARGMAX_SLICES + slice] = best_i;
    }
}

// one warp per row picks among the slices' results
__global__ void __launch_bounds__(32)
argmax_finish_kernel(const float* __restrict__ slice_val, const int* __restrict__ slice_idx, int* __restrict__ out) {
    after_previous_kernel();
    const int row = blockIdx.x, lane = threadIdx.x;
    float best = slice_val[row * ARGMAX_SLICES + lane];
    int best_i = slice_idx[row * ARGMAX_SLICES + lane];
    if (best_i < 0) best = -INFINITY;                                  // a slice of nothing comparable
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        keep_larger(best, best_i, ov, oi);
    }
    if (lane == 0) out[row] = best_i < 0 ? 0 : best_i;
}

// logits [rows, vocab] float32 -> out[r] = the index of row r's largest logit (the last one on ties, 0 if nothing
// compares).  slice_val, slice_idx: scratch of rows * 32 elements each.
FRB_API int frb_argmax_rows(const float* logits, int rows, int vocab, float* slice_val, int* slice_idx, int* out,
                            cudaStream_t stream) {
    if (rows == 0) return 0;
    FRB_CHECK_ARG(vocab >= 1 && rows <= 65535, "argmax: %d rows of %d", rows, vocab);
    launch_dependent_resident(8, argmax_slices_kernel, dim3(ARGMAX_SLICES, rows), dim3(ARGMAX_BLOCK), 0, stream, logits, vocab,
                              slice_val, slice_idx);
    launch_dependent(argmax_finish_kernel, dim3(rows), dim3(32), 0, stream, (const float*)slice_val, (const int*)slice_idx, out);
    FRB_RETURN_LAUNCH("argmax_rows");
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
// Every warp keeps a histogram of its own in shared memory and adds to it without atomic operations: the lanes
// that fall into one value find one another with a match, their counts and weights are added across the
// lanes, and the lowest of them stores the sums (atomic additions of all threads to a few hot values, the
// leading bits of most logits being the same, took 2.5 ms for a vocabulary of 200,064).
// Neither has a counterpart in the reference, which is greedy only (src/minimax.rs:375).
__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_floor_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                    const int* __restrict__ top_k, const float* __restrict__ top_p, float* __restrict__ floor,
                    unsigned int* __restrict__ row_top, unsigned int* __restrict__ first_count,
                    unsigned long long* __restrict__ first_mass) {
    after_previous_kernel();
    constexpr int WARPS = SAMPLE_BLOCK / 32;
    extern __shared__ __align__(16) unsigned char floor_sm[];
    unsigned long long* warp_mass = reinterpret_cast<unsigned long long*>(floor_sm);       // [WARPS][256]
    unsigned int* warp_count = reinterpret_cast<unsigned int*>(warp_mass + WARPS * 256);   // [WARPS][256]
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
    // The row's largest logit and the first histogram, over all logits, come from the two kernels before this one
    // where the vocabulary is large (many blocks per row); else they are made here.
    float top = -INFINITY;
    if (row_top) {
        top = sample_unkey(row_top[row]);
    } else {
        for (int i = threadIdx.x; i < vocab; i += SAMPLE_BLOCK) top = fmaxf(top, x[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
        if (lane == 0) s_red[warp] = top;
        __syncthreads();
        top = s_red[0];
        for (int w = 1; w < 32; ++w) top = fmaxf(top, s_red[w]);
    }
    const float inv_t = 1.0f / temp;
    const float unit = (float)(1ull << SAMPLE_MASS_BITS);
    if (threadIdx.x == 0) {
        s_prefix = 0;
        s_want_count = k > 0 ? (unsigned int)k : 0xffffffffu;
        s_want_mass = 0;
    }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
        const bool given = shift == 24 && first_count != nullptr;
        for (int i = threadIdx.x; i < WARPS * 256; i += SAMPLE_BLOCK) { warp_count[i] = 0; warp_mass[i] = 0; }
        __syncthreads();
        const unsigned int prefix = s_prefix;
        const unsigned int above = shift == 24 ? 0u : 0xffffffffu << (shift + 8);      // the bits found so far
        unsigned int* my_count = warp_count + warp * 256;
        unsigned long long* my_mass = warp_mass + warp * 256;
        // eight loads are on their way at a time: a trip that waits for one load at a time is bound by the memory's
        // latency (32 warps x 128 bytes in flight), not by its instructions
        constexpr int AHEAD = 8;
        for (int first = warp * 32; first < vocab && !given; first += AHEAD * SAMPLE_BLOCK) {    // the same trips for every lane
            float ahead[AHEAD];
#pragma unroll
            for (int a = 0; a < AHEAD; ++a) {
                const int i = first + a * SAMPLE_BLOCK + lane;
                ahead[a] = i < vocab ? x[i] : 0.f;
            }
#pragma unroll
            for (int a = 0; a < AHEAD; ++a) {
                const int i = first + a * SAMPLE_BLOCK + lane;
                const float v = ahead[a];
                const unsigned int key = sample_key(v);
                const bool mine = i < vocab && (key & above) == prefix;
                // no logit of the warp takes part any more in most trips of the later passes
                const unsigned int taking_part = __ballot_sync(0xffffffffu, mine);
                if (!taking_part) continue;
                const unsigned int digit = mine ? (key >> shift) & 255u : 256u;           // the others share a value of their own
                const unsigned long long mass = mine ? (unsigned long long)(expf((v - top) * inv_t) * unit) : 0ull;
                if (__popc(taking_part) <= 6) {
                    // a few lanes: one after the other (a match costs a round for every value that occurs)
                    for (unsigned int rest = taking_part; rest; rest &= rest - 1) {
                        if (lane == __ffs(rest) - 1) { my_count[digit] += 1; my_mass[digit] += mass; }
                        __syncwarp();
                    }
                    continue;
                }
                const unsigned int same = __match_any_sync(0xffffffffu, digit);
                // at most 2^40 each: the halves of 20 bits add up over 32 lanes within 32 bits
                const unsigned int low = __reduce_add_sync(same, (unsigned int)(mass & 0xfffffu));
                const unsigned int high = __reduce_add_sync(same, (unsigned int)(mass >> 20));
                if (mine && lane == __ffs(same) - 1) {
                    my_count[digit] += __popc(same);
                    my_mass[digit] += ((unsigned long long)high << 20) + low;
                }
                __syncwarp();
            }
        }
        __syncthreads();
        for (int d = threadIdx.x; d < 256; d += SAMPLE_BLOCK) {
            unsigned int count = 0;
            unsigned long long mass = 0;
            if (given) {
                count = first_count[(size_t)row * 256 + d];
                mass = first_mass[(size_t)row * 256 + d];
                first_count[(size_t)row * 256 + d] = 0;              // zero again for the next call
                first_mass[(size_t)row * 256 + d] = 0;
            } else {
                for (int w = 0; w < WARPS; ++w) { count += warp_count[w * 256 + d]; mass += warp_mass[w * 256 + d]; }
            }
            s_count[d] = count;
            s_mass[d] = mass;
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
    }
    if (threadIdx.x == 0) {
        floor[row] = sample_unkey(s_prefix);
        if (row_top) row_top[row] = 0;                                // zero again for the next call
    }
}

// The two kernels that go before sample_floor_kernel where a row is worth many blocks: the row's largest logit
// (as an ordered key, by an atomic maximum), then the histogram over the leading eight bits of every logit, each
// block adding its slice's counts and weights (integers) to the row's.  Rows that cut nothing are left out.
__device__ __forceinline__ bool floor_cuts(const float* temperature, const int* top_k, const float* top_p, int row) {
    const float temp = temperature ? temperature[row] : 0.f;
    return temp > 0.f && ((top_k && top_k[row] > 0) || (top_p && top_p[row] < 1.f));
}

__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_floor_top_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                        const int* __restrict__ top_k, const float* __restrict__ top_p, unsigned int* __restrict__ row_top) {
    after_previous_kernel();
    __shared__ float s_red[32];
    const int row = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (!floor_cuts(temperature, top_k, top_p, row)) return;
    const float* x = logits + (size_t)row * vocab;
    float top = -INFINITY;
    for (int i = blockIdx.x * SAMPLE_BLOCK + threadIdx.x; i < vocab; i += gridDim.x * SAMPLE_BLOCK) top = fmaxf(top, x[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    if (lane == 0) s_red[warp] = top;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SAMPLE_BLOCK / 32; ++w) top = fmaxf(top, s_red[w]);
        atomicMax(&row_top[row], sample_key(top));
    }
}

__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_floor_first_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                          const int* __restrict__ top_k, const float* __restrict__ top_p,
                          const unsigned int* __restrict__ row_top, unsigned int* __restrict__ first_count,
                          unsigned long long* __restrict__ first_mass) {
    after_previous_kernel();
    constexpr int WARPS = SAMPLE_BLOCK / 32;
    extern __shared__ __align__(16) unsigned char floor_sm[];
    unsigned long long* warp_mass = reinterpret_cast<unsigned long long*>(floor_sm);       // [WARPS][256]
    unsigned int* warp_count = reinterpret_cast<unsigned int*>(warp_mass + WARPS * 256);   // [WARPS][256]
    const int row = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (!floor_cuts(temperature, top_k, top_p, row)) return;
    const float* x = logits + (size_t)row * vocab;
    const float top = sample_unkey(row_top[row]);
    const float inv_t = 1.0f / temperature[row];
    const float unit = (float)(1ull << SAMPLE_MASS_BITS);
    for (int i = threadIdx.x; i < WARPS * 256; i += SAMPLE_BLOCK) { warp_count[i] = 0; warp_mass[i] = 0; }
    __syncthreads();
    unsigned int* my_count = warp_count + warp * 256;
    unsigned long long* my_mass = warp_mass + warp * 256;
    for (int base = blockIdx.x * SAMPLE_BLOCK + warp * 32; base < vocab; base += gridDim.x * SAMPLE_BLOCK) {
        const int i = base + lane;
        const bool mine = i < vocab;
        const float v = mine ? x[i] : 0.f;
        const unsigned int digit = mine ? sample_key(v) >> 24 : 256u;
        const unsigned int same = __match_any_sync(0xffffffffu, digit);
        const unsigned long long mass = mine ? (unsigned long long)(expf((v - top) * inv_t) * unit) : 0ull;
        const unsigned int low = __reduce_add_sync(same, (unsigned int)(mass & 0xfffffu));
        const unsigned int high = __reduce_add_sync(same, (unsigned int)(mass >> 20));
        if (mine && lane == __ffs(same) - 1) {
            my_count[digit] += __popc(same);
            my_mass[digit] += ((unsigned long long)high << 20) + low;
        }
        __syncwarp();
    }
    __syncthreads();
    for (int d = threadIdx.x; d < 256; d += SAMPLE_BLOCK) {
        unsigned int count = 0;
        unsigned long long mass = 0;
        for (int w = 0; w < WARPS; ++w) { count += warp_count[w * 256 + d]; mass += warp_mass[w * 256 + d]; }
        if (count) {
            atomicAdd(&first_count[(size_t)row * 256 + d], count);
            atomicAdd(&first_mass[(size_t)row * 256 + d], mass);
        }
    }
}

// floor[row] = the smallest logit of the row that sampling may pick (see the kernel); -inf where the row is
// greedy or neither top_k (> 0) nor top_p (< 1) cuts anything.  top_k, top_p: [rows] or null.
FRB_API int frb_sample_floor(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                             const float* top_p, float* floor, unsigned int* row_top, unsigned int* first_count,
                             unsigned long long* first_mass, cudaStream_t stream) {
    if (rows == 0) return 0;
    FRB_CHECK_ARG(vocab >= 1, "sampling: a vocabulary of %d", vocab);
    FRB_CHECK_ARG(rows <= 65535, "sampling: %d rows exceed the grid", rows);
    const size_t smem = (size_t)(SAMPLE_BLOCK / 32) * 256 * (sizeof(unsigned long long) + sizeof(unsigned int));
    cudaFuncSetAttribute(sample_floor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // row_top [rows], first_count [rows, 256], first_mass [rows, 256]: scratch that is zero before the call and is left
    // zero; with it, and a vocabulary worth several blocks a row, the passes over every logit are spread over the SMs
    const int slices = vocab / (8 * SAMPLE_BLOCK) < 32 ? vocab / (8 * SAMPLE_BLOCK) : 32;
    if (row_top && first_count && first_mass && slices >= 2) {
        cudaFuncSetAttribute(sample_floor_first_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(sample_floor_top_kernel, dim3(slices, rows), dim3(SAMPLE_BLOCK), 0, stream, logits, vocab, temperature, top_k,
                         top_p, row_top);
        launch_dependent(sample_floor_first_kernel, dim3(slices, rows), dim3(SAMPLE_BLOCK), smem, stream, logits, vocab, temperature,
                         top_k, top_p, (const unsigned int*)row_top, first_count, first_mass);
        launch_dependent(sample_floor_kernel, dim3(rows), dim3(SAMPLE_BLOCK), smem, stream, logits, vocab, temperature, top_k, top_p,
                         floor, row_top, first_count, first_mass);
    } else {
        launch_dependent(sample_floor_kernel, dim3(rows), dim3(SAMPLE_BLOCK), smem, stream, logits, vocab, temperature, top_k, top_p,
                         floor, (unsigned int*)nullptr, (unsigned int*)nullptr, (unsigned long long*)nullptr);
    }
    FRB_RETURN_LAUNCH("sample_floor");
}
