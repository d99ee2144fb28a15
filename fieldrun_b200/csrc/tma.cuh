// Tensor-map copies into shared memory and the mbarriers that announce them.
//
// A wait on an mbarrier gives up after about a second, or at once when another wait of the block has given
// up: it then sets the block's `failed` flag and returns false, so that no block spins for ever.
#pragma once

#include <cuda.h>

#include "common.cuh"

#define FRB_TMA_WAIT_CYCLES (2000000000ll)

namespace frb_tma {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

// makes freshly initialised barriers known to the unit that completes the copies
__device__ __forceinline__ void bar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool bar_try(uint32_t addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    return done != 0;
}

// Waits for the phase of the given parity.  The clock and the block's flag are only looked at when the
// phase is not complete at the first try: most waits of a running pipeline are.
// `limit`: clock cycles after which the wait gives up (about a second by default).
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* failed,
                                         long long limit = FRB_TMA_WAIT_CYCLES) {
    const uint32_t addr = smem_addr(bar);
    if (bar_try(addr, parity)) return true;
    const long long start = clock64();
    for (;;) {
        if (bar_try(addr, parity)) return true;
        if (*failed || clock64() - start > limit) { *failed = 1; return false; }
    }
}

// one box of the tensor map, its first element at column x of row y, into dst; the bytes count on `bar`
__device__ __forceinline__ void load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}

// one box of a five-dimensional tensor map, its first element at the given coordinates (innermost first), with a
// cache policy for L2 (see createpolicy)
__device__ __forceinline__ void load_5d_hint(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar,
                                             uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(policy) : "memory");
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeFn encoder() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = (EncodeFn)ptr;
    }
    return fn;
}

// A map over row-major bfloat16 [rows, cols] with boxes of [box_rows, 64 columns] (rows of 128 bytes in
// shared memory, 128-byte swizzle: the 16-byte chunk c of row r lies at chunk c ^ (r & 7)); zeros outside.
static inline bool map_rows_of_64(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeFn fn = encoder();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A map over row-major bfloat16 weights for the kernel that streams them, sixteen rows at a time.  The sixteen
// rows are two runs of eight (`half_stride` elements apart: the next eight rows, or the same eight features of
// the second matrix of a pair); a group of sixteen follows the one before it `group_stride` elements on.  The
// inner size is cut into pieces of 64 (128 bytes), so that a box lies in shared memory as
// [piece][run][row of eight][64] with the 128-byte swizzle (chunk c of row r at chunk c ^ r).
// Coordinates: (0, 0, 0, first piece, group); `pieces` pieces per box.  The inner size is a multiple of 64.
static inline bool map_rows_in_pieces(CUtensorMap* map, const void* base, uint64_t inner, uint64_t half_stride,
                                      uint64_t group_stride, uint64_t groups, uint32_t pieces) {
    EncodeFn fn = encoder();
    if (!fn) return false;
    cuuint64_t dims[5] = {64, 8, 2, inner / 64, groups};
    cuuint64_t strides[4] = {inner * 2, half_stride * 2, 128, group_stride * 2};
    cuuint32_t box[5] = {64, 8, 2, pieces, 1};
    cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace frb_tma
