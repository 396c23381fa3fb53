// Decode attention (one new token per sequence) over the paged cache, fast form.
//
// grid = (splits, kv_heads, sequences).  A block of W warps handles W pages
// (64 positions each) of one sequence and kv head, for all query heads of that
// kv head.  One thread starts bulk copies (cp.async.bulk, completion on an
// mbarrier) of the pages' key and value tiles — each tile is one contiguous
// [64][head_dim] block of the cache — so that everything the block needs is in
// flight at once; scores, softmax statistics and the weighted sum of values are
// then computed from shared memory in float32.  A second kernel merges the
// splits of a sequence in index order.  The plain form of the same computation
// (global loads, no shared-memory staging) is attn_decode_kernel in attn.cu.
//
// Formulas: wick src/model.rs:520-553 (see attn.cu).  The split size is fixed by
// the head size and the element type, the order of every sum is fixed, so a
// sequence's result does not depend on what else is in the batch.
#include "common.cuh"
#include "sm100.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace fastdecode {

constexpr int HD = WICK_HD;
constexpr int GT = 4;                                  // query heads handled per pass

template <typename T> struct Shape {
    static constexpr int EPC = Vec16<T>::N;                      // elements per 16-byte chunk
    static constexpr int CHUNKS = HD / EPC;                      // chunks per row
    static constexpr int TILE_BYTES = kPage * HD * (int)sizeof(T);
    static constexpr int W_RAW = 65536 / (2 * TILE_BYTES);
    static constexpr int WARPS = W_RAW >= 4 ? 4 : (W_RAW >= 2 ? 2 : 1);
    static constexpr int SPLIT = WARPS * kPage;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int pow2ceil(int v) { int p = 1; while (p < v) p <<= 1; return p; }
    static constexpr int TS = CHUNKS >= 32 ? 32 : pow2ceil(CHUNKS);   // lanes that share a key in the value pass
    static constexpr int CPL = (CHUNKS + TS - 1) / TS;
    static constexpr int KPI = 32 / TS;
    static constexpr bool SWZ = CHUNKS % 8 == 0;                 // visit chunks in a per-lane order that avoids bank conflicts
    static constexpr size_t SMEM = (size_t)2 * WARPS * TILE_BYTES + (size_t)(GT * HD + GT * SPLIT + WARPS * GT * HD) * sizeof(float);
};

template <typename T>
__global__ void __launch_bounds__(Shape<T>::THREADS)
attn_decode_fast_kernel(const T* __restrict__ q, const T* __restrict__ kv, float* __restrict__ part_o,
                        float* __restrict__ part_ml, const int* __restrict__ kv_len_arr,
                        const int* __restrict__ page_table, int table_width, int n_heads, int n_kv, int max_splits,
                        float scale, int* status) {
    using S = Shape<T>;
    constexpr int EPC = S::EPC, CHUNKS = S::CHUNKS, WARPS = S::WARPS, SPLIT = S::SPLIT, THREADS = S::THREADS;
    constexpr int TS = S::TS, CPL = S::CPL, KPI = S::KPI;
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    kv = fresh(kv);
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    // A length beyond what the page table or the scratch (max_splits) holds is cut back to it
    // and reported: nothing outside the table or the scratch is touched.
    const int most = min(table_width * kPage, max_splits * SPLIT);
    int kv_len = kv_len_arr[b];
    if (kv_len > most) {
        if (split == 0 && kvh == 0 && threadIdx.x == 0 && status) atomicCAS(status, 0, 10);
        kv_len = most;
    }
    const int key_begin = split * SPLIT;
    if (key_begin >= kv_len) return;
    const int group = n_heads / n_kv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    extern __shared__ __align__(128) uint8_t smem_raw[];
    T* k_s = reinterpret_cast<T*>(smem_raw);                               // [WARPS][64][HD]
    T* v_s = k_s + (size_t)WARPS * kPage * HD;                             // [WARPS][64][HD]
    float* q_s = reinterpret_cast<float*>(v_s + (size_t)WARPS * kPage * HD);   // [GT][HD]
    float* sc = q_s + GT * HD;                                             // [GT][SPLIT]
    float* red = sc + GT * SPLIT;                                          // [WARPS][GT][HD]
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    __shared__ float stat[GT][2];
    __shared__ float scratch[40];

    const int n_pages = min(WARPS, (kv_len - key_begin + kPage - 1) / kPage);
    if (tid == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        const int64_t page_elems = (int64_t)2 * n_kv * kPage * HD;
        mbar_expect_tx(&bar, (uint32_t)(2 * n_pages * S::TILE_BYTES));
        for (int w = 0; w < n_pages; ++w) {
            const int page = page_table[(int64_t)b * table_width + key_begin / kPage + w];
            const T* kp = kv + page * page_elems + ((int64_t)kvh * kPage) * HD;
            bulk_load(k_s + (size_t)w * kPage * HD, kp, S::TILE_BYTES, &bar);
            bulk_load(v_s + (size_t)w * kPage * HD, kp + (int64_t)n_kv * kPage * HD, S::TILE_BYTES, &bar);
        }
    }
    const bool warp_live = warp < n_pages;
    const T* kw = k_s + (size_t)warp * kPage * HD;
    const T* vw = v_s + (size_t)warp * kPage * HD;
    bool waited = false;

    for (int h0 = 0; h0 < group; h0 += GT) {
        const int nh = min(GT, group - h0);
        __syncthreads();
        for (int i = tid; i < GT * HD; i += THREADS) {
            const int h = i / HD, d = i % HD;
            q_s[i] = h < nh ? ld(q + ((int64_t)b * n_heads + kvh * group + h0 + h) * HD + d) : 0.f;
        }
        __syncthreads();
        if (!waited) {
            mbar_wait(&bar, 0, &abort_flag, status, 4);
            waited = true;
            __syncthreads();
            if (abort_flag) break;          // the same decision in every thread
        }

        // ---- scores: lane = key (two keys per lane), chunks of the row in turn ----
        float s[2][GT];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int h = 0; h < GT; ++h) s[kk][h] = 0.f;
        if (warp_live) {
#pragma unroll 2
            for (int c = 0; c < CHUNKS; ++c) {
                const int cc = S::SWZ ? (c ^ (lane & 7)) : c;
                Vec16<T> k0, k1;
                k0.load(kw + (size_t)lane * HD + cc * EPC);
                k1.load(kw + (size_t)(lane + 32) * HD + cc * EPC);
#pragma unroll
                for (int h = 0; h < GT; ++h) {
                    const float* qh = q_s + h * HD + cc * EPC;
#pragma unroll
                    for (int e = 0; e < EPC; e += 4) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qh + e);
                        s[0][h] = fmaf(q4.x, k0.v[e], s[0][h]); s[0][h] = fmaf(q4.y, k0.v[e + 1], s[0][h]);
                        s[0][h] = fmaf(q4.z, k0.v[e + 2], s[0][h]); s[0][h] = fmaf(q4.w, k0.v[e + 3], s[0][h]);
                        s[1][h] = fmaf(q4.x, k1.v[e], s[1][h]); s[1][h] = fmaf(q4.y, k1.v[e + 1], s[1][h]);
                        s[1][h] = fmaf(q4.z, k1.v[e + 2], s[1][h]); s[1][h] = fmaf(q4.w, k1.v[e + 3], s[1][h]);
                    }
                }
            }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const int key = lane + 32 * kk;
            const bool valid = warp_live && key_begin + warp * kPage + key < kv_len;
#pragma unroll
            for (int h = 0; h < GT; ++h) sc[h * SPLIT + warp * kPage + key] = valid ? s[kk][h] * scale : -INFINITY;
        }
        __syncthreads();

        // ---- softmax statistics of the split, per head (each thread owns two scores) ----
        for (int h = 0; h < GT; ++h) {
            float m = fmaxf(sc[h * SPLIT + tid], sc[h * SPLIT + tid + THREADS]);
            m = warp_max(m);
            if (lane == 0) scratch[warp] = m;
            __syncthreads();
            m = scratch[0];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) m = fmaxf(m, scratch[w]);
            const float p0 = expf(sc[h * SPLIT + tid] - m), p1 = expf(sc[h * SPLIT + tid + THREADS] - m);
            const float l = block_sum(p0 + p1, scratch + 4);
            sc[h * SPLIT + tid] = p0;
            sc[h * SPLIT + tid + THREADS] = p1;
            if (tid == 0) { stat[h][0] = m; stat[h][1] = l; }
            __syncthreads();
        }

        // ---- weighted sum of values: TS lanes share a key, each owns 16-byte chunks of the row ----
        const int tl = lane % TS, team = lane / TS;
        float acc[GT][CPL][EPC];
#pragma unroll
        for (int h = 0; h < GT; ++h)
#pragma unroll
            for (int c = 0; c < CPL; ++c)
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc[h][c][e] = 0.f;
        if (warp_live) {
            const int keys_here = min(kPage, kv_len - key_begin - warp * kPage);
#pragma unroll 4
            for (int it = 0; it < kPage / KPI; ++it) {
                const int key = it * KPI + team;
                if (key < keys_here) {
#pragma unroll
                    for (int c = 0; c < CPL; ++c) {
                        const int chunk = tl + c * TS;
                        if (chunk < CHUNKS) {
                            Vec16<T> vv;
                            vv.load(vw + (size_t)key * HD + chunk * EPC);
#pragma unroll
                            for (int h = 0; h < GT; ++h) {
                                const float p = sc[h * SPLIT + warp * kPage + key];
#pragma unroll
                                for (int e = 0; e < EPC; ++e) acc[h][c][e] = fmaf(p, vv.v[e], acc[h][c][e]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int h = 0; h < GT; ++h)
#pragma unroll
            for (int c = 0; c < CPL; ++c)
#pragma unroll
                for (int e = 0; e < EPC; ++e) {
                    float v = acc[h][c][e];
#pragma unroll
                    for (int o = TS; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    const int chunk = tl + c * TS;
                    if (team == 0 && chunk < CHUNKS) red[(warp * GT + h) * HD + chunk * EPC + e] = v;
                }
        __syncthreads();
        for (int i = tid; i < nh * HD; i += THREADS) {
            const int h = i / HD, d = i % HD;
            float v = red[h * HD + d];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) v += red[(w * GT + h) * HD + d];
            const int64_t row = ((int64_t)b * n_heads + kvh * group + h0 + h) * max_splits + split;
            part_o[row * HD + d] = v;
            if (d == 0) {
                part_ml[row * 2] = stat[h][0];
                part_ml[row * 2 + 1] = stat[h][1];
            }
        }
    }
    if (!waited) mbar_wait(&bar, 0, &abort_flag, status, 4);     // never leave with copies in flight
    if (abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
}

template <typename T>
__global__ void attn_decode_fast_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ kv_len_arr, T* __restrict__ out, int n_heads,
                                              int max_splits) {
    constexpr int SPLIT = Shape<T>::SPLIT;
    pdl_trigger();
    pdl_wait();
    part_o = fresh(part_o);
    part_ml = fresh(part_ml);
    const int head = blockIdx.x, b = blockIdx.y;
    const int n_splits = min((kv_len_arr[b] + SPLIT - 1) / SPLIT, max_splits);   // (a longer length was cut back and reported)
    const int64_t row0 = ((int64_t)b * n_heads + head) * max_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(row0 + s) * 2]);
    float denom = 0.f;
    for (int s = 0; s < n_splits; ++s) denom += expf(part_ml[(row0 + s) * 2] - m) * part_ml[(row0 + s) * 2 + 1];
    const float inv = n_splits > 0 ? 1.0f / denom : 0.f;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_splits; ++s) v = fmaf(expf(part_ml[(row0 + s) * 2] - m), part_o[(row0 + s) * HD + d], v);
        st(out + ((int64_t)b * n_heads + head) * HD + d, v * inv);
    }
}

template <typename T>
int run(const void* q, const void* kv, void* out, float* scratch, int64_t scratch_floats, const int* kv_len, int n_seqs,
        int max_kv_len, const int* page_table, int table_width, int n_heads, int n_kv, float scale, int* status,
        cudaStream_t s) {
    using S = Shape<T>;
    WICK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads over %d kv heads", n_heads, n_kv);
    WICK_REQUIRE(n_kv <= 65535 && n_seqs <= 65535, "attention: grid limit");
    if (n_seqs == 0) return 0;
    const int max_splits = ceil_div(max_kv_len > 0 ? max_kv_len : 1, S::SPLIT);
    const int64_t need = (int64_t)n_seqs * n_heads * max_splits * (HD + 2);
    WICK_REQUIRE(scratch_floats >= need, "attention decode: scratch of %lld floats, %lld needed",
                 (long long)scratch_floats, (long long)need);
    float* ml = scratch + (int64_t)n_seqs * n_heads * max_splits * HD;
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_fast_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
        raised = true;
    }
    WICK_CUDA(launch(attn_decode_fast_kernel<T>, dim3(max_splits, n_kv, n_seqs), dim3(S::THREADS), S::SMEM, s, (const T*)q,
                     (const T*)kv, scratch, ml, kv_len, page_table, table_width, n_heads, n_kv, max_splits, scale, status));
    if (int e = check_launch("attn_decode")) return e;
    WICK_CUDA(launch(attn_decode_fast_merge_kernel<T>, dim3(n_heads, n_seqs), dim3(HD >= 128 ? 128 : 64), 0, s,
                     (const float*)scratch, (const float*)ml, kv_len, (T*)out, n_heads, max_splits));
    return check_launch("attn_decode_merge");
}

}  // namespace fastdecode
}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

// Positions per split of the fast decode kernels (the scratch holds, per
// sequence and head, ceil(max_kv_len / split) partial results of HD + 2 floats).
WICK_API int wick_attn_decode_split_bf16() { return fastdecode::Shape<bf16>::SPLIT; }
WICK_API int wick_attn_decode_split_f32() { return fastdecode::Shape<float>::SPLIT; }

// q, out: [n_seqs, n_heads, HD]; kv: one schedule entry's cache.  status: device
// int that receives 4 if a block gave up waiting for its copies, 10 if a length was beyond the
// page table or max_kv_len (it is then cut back to what they hold).
WICK_API int wick_attn_decode_bf16(const void* q, const void* kv, void* out, float* scratch, int64_t scratch_floats,
                                   const int* kv_len, int n_seqs, int max_kv_len, const int* page_table,
                                   int table_width, int n_heads, int n_kv, float scale, int* status, void* s) {
    return fastdecode::run<bf16>(q, kv, out, scratch, scratch_floats, kv_len, n_seqs, max_kv_len, page_table, table_width,
                                 n_heads, n_kv, scale, status, (cudaStream_t)s);
}
WICK_API int wick_attn_decode_f32(const void* q, const void* kv, void* out, float* scratch, int64_t scratch_floats,
                                  const int* kv_len, int n_seqs, int max_kv_len, const int* page_table,
                                  int table_width, int n_heads, int n_kv, float scale, int* status, void* s) {
    return fastdecode::run<float>(q, kv, out, scratch, scratch_floats, kv_len, n_seqs, max_kv_len, page_table, table_width,
                                  n_heads, n_kv, scale, status, (cudaStream_t)s);
}

// ---------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory (declared in
// attn_decode_noalloc.h; wick has nothing like it).
//
// wick_attn_decode_bf16 above needs a scratch buffer from its caller for the
// per-split partial results.  A host that has no allocator to ask — a plug-in
// inside another runtime's memory pool, a real-time loop that may not block in
// cudaMalloc, a process whose memory budget is fixed at load time — can call
// this entry point instead: the partial results go to a fixed array that is part
// of this library's image on the device.
//
// * The array holds kNoAllocFloats float32 (8 MiB).  Every GPU that loads this
//   library carries it until the process exits.  A call that needs more
//   (n_seqs * n_heads * ceil(max_kv_len / split) * (head_dim + 2) floats) is
//   refused with an error; nothing is launched.
// * In host code the array's name is only a handle.  The device address is
//   looked up with cudaGetSymbolAddress, once per device, by the first call made
//   while that device is current; make that first call before capturing a stream.
// * All calls share the one array, and it keeps what the last call left.  Nothing
//   in it has to start at zero: every entry a call reads was written by that
//   call.  Two calls that overlap on the GPU (different streams) race on it; keep
//   calls that use this entry point on one stream or order them with events.
// * No cudaMalloc, cudaFree or other allocating routine is called, here or below.
namespace wick {
namespace fastdecode {

constexpr long long kNoAllocFloats = 2ll * 1024 * 1024;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

static int noalloc_scratch(float** out) {
    // (No lock: two host threads may both look the symbol up on a device's first call; they
    // store the same address.)
    static float* per_device[64] = {};
    int dev = -1;
    WICK_CUDA(cudaGetDevice(&dev));
    WICK_REQUIRE(dev >= 0 && dev < 64, "attention decode (no allocation): device index %d is out of range", dev);
    if (per_device[dev] == nullptr) {
        float* p = nullptr;
        WICK_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
        WICK_REQUIRE(p != nullptr, "attention decode (no allocation): the scratch array has no device address");
        per_device[dev] = p;
    }
    *out = per_device[dev];
    return 0;
}

}  // namespace fastdecode
}  // namespace wick

WICK_API long long wick_attn_decode_noalloc_capacity() { return wick::fastdecode::kNoAllocFloats; }

WICK_API int wick_attn_decode_noalloc_bf16(const void* q, const void* kv, void* out, const int* kv_len, int n_seqs,
                                           int max_kv_len, const int* page_table, int table_width, int n_heads,
                                           int n_kv, float scale, int* status, void* s) {
    using namespace wick::fastdecode;
    WICK_REQUIRE(n_seqs >= 0 && n_heads > 0 && max_kv_len >= 0, "attention decode (no allocation): bad sizes");
    const long long splits = (max_kv_len > 0 ? max_kv_len : 1) / Shape<bf16>::SPLIT +
                             ((max_kv_len > 0 ? max_kv_len : 1) % Shape<bf16>::SPLIT != 0);
    const long long need = (long long)n_seqs * n_heads * splits * (HD + 2);
    WICK_REQUIRE(need <= kNoAllocFloats,
                 "attention decode (no allocation): %d sequences x %d heads x %lld splits need %lld floats of scratch, "
                 "the built-in array holds %lld", n_seqs, n_heads, splits, need, kNoAllocFloats);
    float* scratch = nullptr;
    if (int e = noalloc_scratch(&scratch)) return e;
    return run<bf16>(q, kv, out, scratch, kNoAllocFloats, kv_len, n_seqs, max_kv_len, page_table, table_width, n_heads,
                     n_kv, scale, status, (cudaStream_t)s);
}
