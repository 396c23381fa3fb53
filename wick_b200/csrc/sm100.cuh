// Thin wrappers over the sm_100a PTX that several kernel files share: shared
// memory addresses, mbarriers with a bounded wait, and the untiled bulk copy.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace wick {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false (and raises the block's abort flag) after limit_ns (~1 s).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          uint64_t limit_ns = 1000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;         // the common case costs one instruction
    if (*abort_flag) return false;
    const uint64_t t0 = global_ns();
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// global -> shared copy of `bytes` contiguous bytes (both addresses 16-byte
// aligned, bytes a multiple of 16); completion is counted on the mbarrier.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Tiled TMA load of one box of a 2-D tensor map; x is the inner coordinate (its
// byte offset must be a multiple of 16), completion is counted on the mbarrier.
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, cols] bfloat16 matrix, row-major, as a TMA descriptor with boxes of
// box_rows x 64 elements (128 bytes, the width of the 128-byte swizzle).
inline int make_bf16_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int box_rows, const char* who) {
    EncodeTiledFn fn = encode_tiled_fn();
    WICK_REQUIRE(fn != nullptr, "%s: the driver does not provide cuTensorMapEncodeTiled", who);
    WICK_REQUIRE(((uintptr_t)ptr & 15) == 0, "%s: operand is not 16-byte aligned", who);
    WICK_REQUIRE(cols % 8 == 0, "%s: inner size %lld is not a multiple of 8 (16-byte rows)", who, (long long)cols);
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    WICK_REQUIRE(r == CUDA_SUCCESS, "%s: cuTensorMapEncodeTiled failed with code %d (rows %lld, cols %lld, box %d)", who,
                 (int)r, (long long)rows, (long long)cols, box_rows);
    return 0;
}

}  // namespace wick
