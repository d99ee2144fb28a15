// Shared helpers of the sm_100a kernels: element types, reductions with a fixed order,
// the error string that the C entry points leave for the Python side.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <stdint.h>
#include <stdio.h>

#define FRB_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

// Element type codes used by every entry point.
enum FrbDtype { FRB_F32 = 0, FRB_BF16 = 1 };

// Tokens per cache page; must equal PAGE_TOKENS of the Python cache.
#define FRB_PAGE 64

void frb_set_error(const char* fmt, ...);

#define FRB_CHECK_ARG(cond, ...)            \
    do {                                    \
        if (!(cond)) {                      \
            frb_set_error(__VA_ARGS__);     \
            return -1;                      \
        }                                   \
    } while (0)

#define FRB_RETURN_LAUNCH(name)                                                   \
    do {                                                                          \
        cudaError_t frb_e_ = cudaGetLastError();                                  \
        if (frb_e_ != cudaSuccess) {                                              \
            frb_set_error("%s: launch failed: %s", name, cudaGetErrorString(frb_e_)); \
            return (int)frb_e_;                                                   \
        }                                                                         \
        return 0;                                                                 \
    } while (0)

// Programmatic dependent launch.  A kernel started with launch_dependent() may begin while the kernel before
// it in the stream still runs; it calls after_previous_kernel() before it reads or writes anything, which
// first lets the kernel after it begin in the same way and then waits until the kernel before it has ended
// and its writes are visible.  What the launch hides is the time between one kernel's last block and the next
// kernel's first instruction, which is most of the cost of the small kernels of a decode step.  In a kernel
// that was started in the ordinary way both instructions do nothing.
//
// A kernel may also do work that does not depend on the kernel before it (loading weights) ahead of
// wait_for_previous_kernel().  If it reads, ahead of the wait, what a kernel two or more places before it in the
// stream wrote, then the kernel directly before it must call let_next_kernel_start() only after its own wait.
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_previous_kernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void after_previous_kernel() {
    let_next_kernel_start();
    wait_for_previous_kernel();
}

// The largest grid that is started early: the number of SMs, or FIELDRUN_B200_PDL from the environment
// (0 starts every kernel in the ordinary way).  Blocks that start early settle on whichever SMs have room at
// that moment; a kernel of many blocks that is bound by memory bandwidth then runs from an uneven placement
// and loses more than the early start gains, so only the small kernels are started early.
inline long frb_dependent_launch_blocks() {
    static const long most = [] {
        const char* v = getenv("FIELDRUN_B200_PDL");
        if (v && v[0]) return atol(v);
        int device = 0, sms = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        return (long)sms;
    }();
    return most;
}

// Starts `kernel`, which orders itself behind the kernel before it with the instructions above, early if its grid
// has at most `per_sm` blocks for every SM (all of them must be able to be resident at once).
template <typename... Params, typename... Args>
inline void launch_dependent_resident(int per_sm, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = (long)grid.x * grid.y * grid.z <= per_sm * frb_dependent_launch_blocks() ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

// Starts `kernel`, whose first statement is after_previous_kernel(), early if its grid has at most a block per SM.
template <typename... Params, typename... Args>
inline void launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    launch_dependent_resident(1, kernel, grid, block, smem, stream, args...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of BLOCK threads; every thread gets the result.  The order of additions depends on
// BLOCK only, so a row's sum is the same whatever else the launch holds.  `scratch` holds 32 floats.
// One warp adds the warps' sums: with every thread reading all of them, a block of 1024 threads made a thousand
// shared-memory loads per call, half a microsecond of a decode step's norm.
template <int BLOCK>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();                      // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const float total = warp_sum(lane < BLOCK / 32 ? scratch[lane] : 0.f);
        if (lane == 0) scratch[0] = total;
    }
    __syncthreads();
    return scratch[0];
}

// Two sums at once (the squares of a token's query and key rows).  `scratch` holds 64 floats.
template <int BLOCK>
__device__ __forceinline__ void block_sum_pair(float& a, float& b, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();                      // scratch may still be read from an earlier call
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
        const float total_a = warp_sum(lane < BLOCK / 32 ? scratch[lane] : 0.f);
        const float total_b = warp_sum(lane < BLOCK / 32 ? scratch[32 + lane] : 0.f);
        if (lane == 0) { scratch[0] = total_a; scratch[32] = total_b; }
    }
    __syncthreads();
    a = scratch[0];
    b = scratch[32];
}

// Calls `body` with a value of the element type that `code` names.
#define FRB_DISPATCH_DTYPE(code, T, ...)                          \
    do {                                                          \
        if ((code) == FRB_F32) { typedef float T; __VA_ARGS__; }  \
        else { typedef bf16 T; __VA_ARGS__; }                     \
    } while (0)
