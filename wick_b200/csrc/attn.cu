// Causal grouped-query attention over the paged cache, for one head size
// (WICK_HD, a multiple of 16, set at compile time) and both element types.
//
//   prompt form : any number of new tokens per sequence, after any cached prefix
//   decode form : one new token per sequence, split over the cached positions
//
// Query token i of a sequence stands at position p = start + i and sees the
// cached positions 0..p (wick src/model.rs:520-553): s_j = (q . k_j) * scale,
// w = softmax(s), out = sum_j w_j v_j; query head h reads kv head h / (heads /
// kv_heads).  Scores, the softmax and the weighted sum are float32.  The cache of
// one schedule entry is laid out [page][k|v][kv_head][64 positions][head_dim].
//
// Results do not depend on the batch: a sequence's work is cut by fixed sizes
// (64 query rows, 64 keys per inner step, 256 keys per decode split) and every
// sum runs in a fixed order.
#include "common.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {

constexpr int HD = WICK_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16 in [16, 256]");

// ============================================================================
// Prompt form.  One block (128 threads) per (64-query tile, head).  Thread
// (r = tid/2, part = tid%2) owns query row r: it computes the scores of 32 of
// the tile's 64 keys and accumulates HD/2 of the output dims.
// ============================================================================
constexpr int QT = 64;             // query rows per block, equals the batch's tile size
constexpr int QS = HD + 4;         // padded row stride of the query tile in shared memory
constexpr int HH = HD / 2;

template <typename T>
__device__ __forceinline__ void load_page_tile(const T* __restrict__ src, float* __restrict__ dst, int valid_rows) {
    // [64][HD] elements, contiguous in global memory, to float32 in shared memory.
    // Rows that hold no token yet are not read (their bytes may be anything) and
    // become zeros, so that a zero weight times such a row stays zero.
    constexpr int VN = Vec16<T>::N;
    for (int i = threadIdx.x * VN; i < kPage * HD; i += blockDim.x * VN) {
        Vec16<T> v;
        if (i / HD < valid_rows) {
            v.load(src + i);
        } else {
#pragma unroll
            for (int j = 0; j < VN; ++j) v.v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < VN; ++j) dst[i + j] = v.v[j];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
attn_prompt_kernel(const T* __restrict__ q, const T* __restrict__ kv, T* __restrict__ out,
                   const int* __restrict__ cu_seqlens, int n_seqs, const int* __restrict__ start,
                   const int* __restrict__ page_table, int table_width, int n_heads, int n_kv, float scale) {
    extern __shared__ float smem[];
    float* Qs = smem;                       // [QT][QS]
    float* Ks = Qs + QT * QS;               // [64][HD]
    float* Vs = Ks + kPage * HD;            // [64][HD]

    const int head = blockIdx.y;
    int b, q0;
    find_work_item(cu_seqlens, n_seqs, QT, blockIdx.x, b, q0);
    if (b < 0) return;
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
    const int s0 = start[b];
    const int rows = min(QT, q_len - q0);
    const int kvh = head / (n_heads / n_kv);
    const int tid = threadIdx.x, r = tid >> 1, part = tid & 1;

    // Query tile to shared memory; rows past the end repeat the last valid row
    // (computed, never stored) so that every row has at least one visible key.
    for (int i = tid; i < QT * (HD / 4); i += blockDim.x) {
        const int rr = i / (HD / 4), c = (i % (HD / 4)) * 4;
        const int src_row = min(rr, rows - 1);
        const T* p = q + ((int64_t)(tok0 + q0 + src_row) * n_heads + head) * HD + c;
#pragma unroll
        for (int j = 0; j < 4; ++j) Qs[rr * QS + c + j] = ld(p + j);
    }

    const int my_row = min(r, rows - 1);
    const int my_pos = s0 + q0 + my_row;              // last visible key of this row
    const int last_key = s0 + q0 + rows - 1;          // last key any row of the tile sees
    const int n_ktiles = last_key / kPage + 1;

    float acc[HH];
#pragma unroll
    for (int d = 0; d < HH; ++d) acc[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int64_t page_elems = (int64_t)2 * n_kv * kPage * HD;

    for (int kt = 0; kt < n_ktiles; ++kt) {
        const int page = page_table[(int64_t)b * table_width + kt];
        const T* kp = kv + page * page_elems + ((int64_t)kvh * kPage) * HD;
        const T* vp = kp + (int64_t)n_kv * kPage * HD;
        __syncthreads();                     // previous tile fully consumed (and Qs written)
        const int valid_rows = s0 + q_len - kt * kPage;   // tokens of this page that the cache holds
        load_page_tile<T>(kp, Ks, valid_rows);
        load_page_tile<T>(vp, Vs, valid_rows);
        __syncthreads();

        // scores of my 32 keys
        float s[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) s[j] = 0.f;
        const float* qrow = Qs + r * QS;
        const float* kbase = Ks + (part * 32) * HD;
#pragma unroll 1
        for (int d0 = 0; d0 < HD; d0 += 8) {
            const float4 qa = *reinterpret_cast<const float4*>(qrow + d0);
            const float4 qb = *reinterpret_cast<const float4*>(qrow + d0 + 4);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float4 ka = *reinterpret_cast<const float4*>(kbase + j * HD + d0);
                const float4 kb = *reinterpret_cast<const float4*>(kbase + j * HD + d0 + 4);
                float t = s[j];
                t = fmaf(qa.x, ka.x, t); t = fmaf(qa.y, ka.y, t); t = fmaf(qa.z, ka.z, t); t = fmaf(qa.w, ka.w, t);
                t = fmaf(qb.x, kb.x, t); t = fmaf(qb.y, kb.y, t); t = fmaf(qb.z, kb.z, t); t = fmaf(qb.w, kb.w, t);
                s[j] = t;
            }
        }
        const int key0 = kt * kPage + part * 32;
        float m_tile = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            s[j] = (key0 + j <= my_pos) ? s[j] * scale : -INFINITY;
            m_tile = fmaxf(m_tile, s[j]);
        }
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
        const float m_new = fmaxf(m_run, m_tile);     // finite: key 0 is visible to every row in tile 0
        const float corr = expf(m_run - m_new);
        float l_tile = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            s[j] = expf(s[j] - m_new);                // masked keys: exp(-inf) = 0
            l_tile += s[j];
        }
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
        l_run = l_run * corr + l_tile;
        m_run = m_new;
#pragma unroll
        for (int d = 0; d < HH; ++d) acc[d] *= corr;

        // acc += P V over the tile's 64 keys, for my HD/2 dims; keys in index order.
#pragma unroll 1
        for (int half_tile = 0; half_tile < 2; ++half_tile) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, s[j], 1);
                const float p = (half_tile == part) ? s[j] : other;
                const float* vrow = Vs + (half_tile * 32 + j) * HD + part * HH;
#pragma unroll
                for (int d = 0; d < HH; d += 4) {
                    const float4 v4 = *reinterpret_cast<const float4*>(vrow + d);
                    acc[d] = fmaf(p, v4.x, acc[d]);
                    acc[d + 1] = fmaf(p, v4.y, acc[d + 1]);
                    acc[d + 2] = fmaf(p, v4.z, acc[d + 2]);
                    acc[d + 3] = fmaf(p, v4.w, acc[d + 3]);
                }
            }
        }
    }
    if (r < rows) {
        const float inv = 1.0f / l_run;
        T* o = out + ((int64_t)(tok0 + q0 + r) * n_heads + head) * HD + part * HH;
#pragma unroll
        for (int d = 0; d < HH; ++d) st(o + d, acc[d] * inv);
    }
}

// ============================================================================
// Decode form.  grid = (splits, kv_heads, sequences); a block handles 256 cached
// positions (one page per warp) for all query heads of its kv head, GT heads at
// a time, and writes unnormalised partial sums with their max and denominator.
// A second kernel merges the splits of a sequence in index order.
// ============================================================================
constexpr int SPLIT = 256;
constexpr int GT = 4;
template <typename T> struct Team {
    static constexpr int EPC = Vec16<T>::N;                      // elements per 16-byte chunk
    static constexpr int CHUNKS = HD / EPC;                      // chunks per row
    static constexpr int pow2ceil(int v) { int p = 1; while (p < v) p <<= 1; return p; }
    static constexpr int SIZE = CHUNKS >= 32 ? 32 : pow2ceil(CHUNKS);   // lanes that share a key
    static constexpr int CPL = (CHUNKS + SIZE - 1) / SIZE;       // chunks per lane
    static constexpr int KEYS = 32 / SIZE;                       // keys per warp iteration
};

template <typename T>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ kv, float* __restrict__ part_o,
                   float* __restrict__ part_ml, const int* __restrict__ kv_len_arr,
                   const int* __restrict__ page_table, int table_width, int n_heads, int n_kv, int max_splits,
                   float scale) {
    using TM = Team<T>;
    constexpr int EPC = TM::EPC, TS = TM::SIZE, CPL = TM::CPL, KPI = TM::KEYS;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int kv_len = kv_len_arr[b];
    const int key_begin = split * SPLIT;
    if (key_begin >= kv_len) return;
    const int group = n_heads / n_kv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tl = lane % TS, team = lane / TS;

    __shared__ float q_s[GT][HD];
    __shared__ float sc[GT][SPLIT];
    __shared__ float red[4][GT][HD];
    __shared__ float stat[GT][2];
    __shared__ float scratch[40];

    const int64_t page_elems = (int64_t)2 * n_kv * kPage * HD;
    const int page_idx = key_begin / kPage + warp;               // this warp's page of the sequence
    const bool warp_live = page_idx * kPage < kv_len;
    const T* kp = nullptr;
    if (warp_live) {
        const int page = page_table[(int64_t)b * table_width + page_idx];
        kp = kv + page * page_elems + ((int64_t)kvh * kPage) * HD;
    }
    const T* vp = kp ? kp + (int64_t)n_kv * kPage * HD : nullptr;

    for (int h0 = 0; h0 < group; h0 += GT) {
        const int nh = min(GT, group - h0);
        __syncthreads();
        for (int i = tid; i < GT * HD; i += blockDim.x) {
            const int h = i / HD, d = i % HD;
            q_s[h][d] = h < nh ? ld(q + ((int64_t)b * n_heads + kvh * group + h0 + h) * HD + d) : 0.f;
        }
        __syncthreads();

        // ---- scores ----
        for (int it = 0; it < kPage / KPI; ++it) {
            const int key = it * KPI + team;
            const int pos = page_idx * kPage + key;
            const bool valid = warp_live && pos < kv_len;
            float part[GT];
#pragma unroll
            for (int h = 0; h < GT; ++h) part[h] = 0.f;
            if (valid) {
#pragma unroll
                for (int c = 0; c < CPL; ++c) {
                    const int chunk = tl + c * TS;
                    if (chunk < TM::CHUNKS) {
                        Vec16<T> kvv;
                        kvv.load(kp + (int64_t)key * HD + chunk * EPC);
#pragma unroll
                        for (int h = 0; h < GT; ++h)
#pragma unroll
                            for (int e = 0; e < EPC; ++e) part[h] = fmaf(q_s[h][chunk * EPC + e], kvv.v[e], part[h]);
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < GT; ++h) {
#pragma unroll
                for (int o = TS / 2; o > 0; o >>= 1) part[h] += __shfl_xor_sync(0xffffffffu, part[h], o);
                if (tl == 0) sc[h][warp * kPage + key] = valid ? part[h] * scale : -INFINITY;
            }
        }
        __syncthreads();

        // ---- softmax statistics of the split, per head ----
        for (int h = 0; h < GT; ++h) {
            float m = fmaxf(sc[h][tid], sc[h][tid + 128]);
            m = warp_max(m);
            if (lane == 0) scratch[warp] = m;
            __syncthreads();
            m = fmaxf(fmaxf(scratch[0], scratch[1]), fmaxf(scratch[2], scratch[3]));
            const float p0 = expf(sc[h][tid] - m), p1 = expf(sc[h][tid + 128] - m);
            const float l = block_sum(p0 + p1, scratch + 4);
            sc[h][tid] = p0;
            sc[h][tid + 128] = p1;
            if (tid == 0) { stat[h][0] = m; stat[h][1] = l; }
            __syncthreads();
        }

        // ---- weighted sum of values ----
        float acc[GT][CPL][EPC];
#pragma unroll
        for (int h = 0; h < GT; ++h)
#pragma unroll
            for (int c = 0; c < CPL; ++c)
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc[h][c][e] = 0.f;
        if (warp_live) {
            for (int it = 0; it < kPage / KPI; ++it) {
                const int key = it * KPI + team;
                if (page_idx * kPage + key < kv_len) {
#pragma unroll
                    for (int c = 0; c < CPL; ++c) {
                        const int chunk = tl + c * TS;
                        if (chunk < TM::CHUNKS) {
                            Vec16<T> vv;
                            vv.load(vp + (int64_t)key * HD + chunk * EPC);
#pragma unroll
                            for (int h = 0; h < GT; ++h) {
                                const float p = sc[h][warp * kPage + key];
#pragma unroll
                                for (int e = 0; e < EPC; ++e) acc[h][c][e] = fmaf(p, vv.v[e], acc[h][c][e]);
                            }
                        }
                    }
                }
            }
        }
        // teams of a warp, then warps, in fixed order
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
                    if (team == 0 && chunk < TM::CHUNKS) red[warp][h][chunk * EPC + e] = v;
                }
        __syncthreads();
        for (int i = tid; i < nh * HD; i += blockDim.x) {
            const int h = i / HD, d = i % HD;
            const float v = ((red[0][h][d] + red[1][h][d]) + red[2][h][d]) + red[3][h][d];
            const int64_t row = ((int64_t)b * n_heads + kvh * group + h0 + h) * max_splits + split;
            part_o[row * HD + d] = v;
            if (d == 0) {
                part_ml[row * 2] = stat[h][0];
                part_ml[row * 2 + 1] = stat[h][1];
            }
        }
    }
}

template <typename T>
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int* __restrict__ kv_len_arr, T* __restrict__ out, int n_heads,
                                         int max_splits) {
    const int head = blockIdx.x, b = blockIdx.y;
    const int n_splits = (kv_len_arr[b] + SPLIT - 1) / SPLIT;
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
int attn_prompt(const void* q, const void* kv, void* out, int n_tiles, const int* cu_seqlens, int n_seqs, const int* start, const int* page_table, int table_width, int n_heads,
                int n_kv, float scale, cudaStream_t s) {
    WICK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads over %d kv heads", n_heads, n_kv);
    WICK_REQUIRE(n_heads <= 65535, "attention: %d heads is beyond the grid limit", n_heads);
    if (n_tiles == 0) return 0;
    const size_t smem = (size_t)(QT * QS + 2 * kPage * HD) * sizeof(float);
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_prompt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised = true;
    }
    attn_prompt_kernel<T><<<dim3(n_tiles, n_heads), 128, smem, s>>>((const T*)q, (const T*)kv, (T*)out, cu_seqlens,
                                                                  n_seqs, start, page_table,
                                                                  table_width, n_heads, n_kv, scale);
    return check_launch("attn_prompt");
}

template <typename T>
int attn_decode(const void* q, const void* kv, void* out, float* part_o, float* part_ml, int64_t scratch_floats,
                const int* kv_len, int n_seqs, int max_kv_len, const int* page_table, int table_width, int n_heads,
                int n_kv, float scale, cudaStream_t s) {
    WICK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads over %d kv heads", n_heads, n_kv);
    WICK_REQUIRE(n_kv <= 65535 && n_seqs <= 65535, "attention: grid limit");
    if (n_seqs == 0) return 0;
    const int max_splits = ceil_div(max_kv_len > 0 ? max_kv_len : 1, SPLIT);
    const int64_t need = (int64_t)n_seqs * n_heads * max_splits * (HD + 2);
    WICK_REQUIRE(scratch_floats >= need, "attention decode: scratch of %lld floats, %lld needed",
                 (long long)scratch_floats, (long long)need);
    (void)part_ml;
    float* ml = part_o + (int64_t)n_seqs * n_heads * max_splits * HD;
    attn_decode_kernel<T><<<dim3(max_splits, n_kv, n_seqs), 128, 0, s>>>(
        (const T*)q, (const T*)kv, part_o, ml, kv_len, page_table, table_width, n_heads, n_kv, max_splits, scale);
    if (int e = check_launch("attn_decode")) return e;
    attn_decode_merge_kernel<T><<<dim3(n_heads, n_seqs), HD >= 128 ? 128 : 64, 0, s>>>(part_o, ml, kv_len, (T*)out,
                                                                                      n_heads, max_splits);
    return check_launch("attn_decode_merge");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

WICK_API int wick_attn_head_dim() { return HD; }
WICK_API int wick_attn_decode_plain_split() { return SPLIT; }

// q, out: [n_tokens, n_heads, HD]; kv: one schedule entry's cache.
WICK_API int wick_attn_prompt_bf16(const void* q, const void* kv, void* out, int n_tiles, const int* cu_seqlens,
                                   int n_seqs, const int* start, const int* page_table,
                                   int table_width, int n_heads, int n_kv, float scale, void* s) {
    return attn_prompt<bf16>(q, kv, out, n_tiles, cu_seqlens, n_seqs, start, page_table, table_width,
                             n_heads, n_kv, scale, (cudaStream_t)s);
}
WICK_API int wick_attn_prompt_f32(const void* q, const void* kv, void* out, int n_tiles, const int* cu_seqlens,
                                  int n_seqs, const int* start, const int* page_table,
                                  int table_width, int n_heads, int n_kv, float scale, void* s) {
    return attn_prompt<float>(q, kv, out, n_tiles, cu_seqlens, n_seqs, start, page_table, table_width,
                              n_heads, n_kv, scale, (cudaStream_t)s);
}
// scratch: float32 [scratch_floats], at least n_seqs*n_heads*ceil(max_kv_len/256)*(HD+2).
WICK_API int wick_attn_decode_plain_bf16(const void* q, const void* kv, void* out, float* scratch, int64_t scratch_floats,
                                   const int* kv_len, int n_seqs, int max_kv_len, const int* page_table,
                                   int table_width, int n_heads, int n_kv, float scale, void* s) {
    return attn_decode<bf16>(q, kv, out, scratch, nullptr, scratch_floats, kv_len, n_seqs, max_kv_len, page_table,
                             table_width, n_heads, n_kv, scale, (cudaStream_t)s);
}
WICK_API int wick_attn_decode_plain_f32(const void* q, const void* kv, void* out, float* scratch, int64_t scratch_floats,
                                  const int* kv_len, int n_seqs, int max_kv_len, const int* page_table,
                                  int table_width, int n_heads, int n_kv, float scale, void* s) {
    return attn_decode<float>(q, kv, out, scratch, nullptr, scratch_floats, kv_len, n_seqs, max_kv_len, page_table,
                              table_width, n_heads, n_kv, scale, (cudaStream_t)s);
}
