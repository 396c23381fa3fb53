// Shared helpers of every kernel file: error reporting over the C ABI, element
// type traits (bfloat16 / float), warp and block reductions.
//
// Every exported function returns 0 on success and a non-zero code otherwise;
// wick_last_error() then returns the message.  Nothing here allocates memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define WICK_API extern "C" __attribute__((visibility("default")))

namespace wick {

inline char* error_buffer() {
    static thread_local char buf[512];
    return buf;
}

inline int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
inline int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return 1;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail("%s: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

#define WICK_REQUIRE(cond, ...)                      \
    do {                                             \
        if (!(cond)) return ::wick::fail(__VA_ARGS__); \
    } while (0)

#define WICK_CUDA(call)                                                          \
    do {                                                                         \
        cudaError_t e_ = (call);                                                 \
        if (e_ != cudaSuccess) return ::wick::fail("%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// ---- element types -------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float ld(const T* p) { return Elem<T>::load(p); }
template <typename T> __device__ __forceinline__ void st(T* p, float v) { Elem<T>::store(p, v); }

// 16-byte vector of elements: 4 floats or 8 bfloat16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        uint4 t = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const {
        uint4 t;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = t;
    }
};

// ---- reductions ------------------------------------------------------------
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

// Sum over the block; every thread gets the result.  scratch: >= 33 floats of
// shared memory.  The order of the additions is fixed by the thread layout.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Positions per cache page.  The Python side carries the same number (wick_b200/layout.py);
// every library exports it (wick_page_size) and the loader refuses a library that differs.
constexpr int kPage = 64;

// The work items of a step whose new tokens are cut into runs of `rows` per sequence are
// numbered sequence by sequence; this finds the sequence b and the first row q0 of item
// `item` from the step's cu_seqlens (which the host writes: no kernel produces it, so it may
// be read before griddepcontrol.wait).  All 32 lanes of the calling warp take part; every
// lane gets the result; b is -1 beyond the last item.
__device__ __forceinline__ void find_work_item(const int* __restrict__ cu_seqlens, int n_seqs, int rows, int item, int& b, int& q0) {
    const int lane = threadIdx.x & 31;
    int before = 0;
    for (int s0 = 0; s0 < n_seqs; s0 += 32) {
        const int s = s0 + lane;
        const int mine = s < n_seqs ? (cu_seqlens[s + 1] - cu_seqlens[s] + rows - 1) / rows : 0;
        int upto = mine;                                         // items of sequences s0 .. s
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, upto, o);
            if (lane >= o) upto += t;
        }
        const int total = __shfl_sync(0xffffffffu, upto, 31);
        if (item < before + total) {
            const unsigned holds = __ballot_sync(0xffffffffu, item - before < upto);
            const int l = __ffs(holds) - 1;
            b = s0 + l;
            q0 = (item - before - __shfl_sync(0xffffffffu, upto - mine, l)) * rows;
            return;
        }
        before += total;
    }
    b = -1;
    q0 = 0;
}

// ---- programmatic dependent launch -------------------------------------------
// Kernels are launched so that the next kernel in the stream may be scheduled
// while this one still runs.  A kernel therefore (1) lets its successor start
// (pdl_trigger) and (2) waits until its predecessor has completed and its writes
// are visible (pdl_wait) before it touches anything another kernel produced or
// may still read.  Only loads of data that no kernel ever writes (weights) may
// come before pdl_wait.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A pointer to data that the kernel before this one produces, as the compiler must
// see it after pdl_wait: a value that exists only from here on.  Without this, a
// load through a const __restrict__ pointer counts as a load of constant data and
// may be moved above the wait (it was, in a kernel whose wait came late: the loads
// then returned what the buffer held before).  Use as: p = fresh(p); right after
// pdl_wait().
template <typename T>
__device__ __forceinline__ T* fresh(T* p) {
    asm volatile("" : "+l"(p));
    return p;
}

// Multiprocessors of the current device (asked once per process and device).
inline int sm_count() {
    static int per_device[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (per_device[dev] == 0) {                        // (two host threads may both ask; they store the same number)
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        per_device[dev] = n;
    }
    return per_device[dev];
}

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("WICK_B200_NO_PDL");
        on = (e && e[0] && e[0] != '0') ? 0 : 1;
    }
    return on == 1;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the programmatic
// serialization attribute (unless WICK_B200_NO_PDL is set).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace wick

// The page size this library was built with.
extern "C" __attribute__((visibility("default"), weak)) int wick_page_size() { return wick::kPage; }

// The message of the last failed call of this library on this thread.
extern "C" __attribute__((visibility("default"), weak)) const char* wick_last_error() { return wick::error_buffer(); }
