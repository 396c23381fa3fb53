// Causal attention of new tokens over the paged cache on the tensor cores
// (bfloat16, head sizes up to 128): the fast form of attn_prompt_kernel in attn.cu,
// with the same work partition (64 query rows x one head per block, one page of
// 64 keys per inner step) and the same float32 softmax.
//
// Four warps of 16 query rows each.  Key and value pages are copied into shared
// memory with cp.async (16 bytes per thread, chunks XOR-swizzled by the row so
// that ldmatrix is free of bank conflicts; rows that hold no token yet are
// zero-filled), two pages deep.  S = Q K^T and O += P V run as mma.sync
// m16n8k16 with float32 accumulators; the running maximum, the denominators and
// the rescaling are float32 in registers.  Scores are multiplied by the scale
// after the dot product (wick src/model.rs:527,538).
#include "common.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace promptmma {

constexpr int HD = WICK_HD;
constexpr int QT = 64;
constexpr int CHUNKS = HD / 8;                       // 16-byte chunks per row
constexpr bool SWZ = CHUNKS % 8 == 0;
constexpr bool SUPPORTED = HD <= 128;
constexpr int KS = HD / 16;                          // k-steps of Q K^T
constexpr int ND = HD / 8;                           // 8-wide blocks of the output row
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ int swz(int row, int chunk) { return SWZ ? (chunk ^ (row & 7)) : chunk; }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One page tile [64][HD] from global (contiguous) into swizzled shared memory.
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src, int valid_rows) {
    for (int i = threadIdx.x; i < kPage * CHUNKS; i += 128) {
        const int row = i / CHUNKS, c = i % CHUNKS;
        cp_async16(dst + row * HD + swz(row, c) * 8, src + row * HD + c * 8, row < valid_rows);
    }
}

__global__ void __launch_bounds__(128)
attn_prompt_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv, bf16* __restrict__ out,
                       const int* __restrict__ cu_seqlens, int n_seqs, const int* __restrict__ start,
                       const int* __restrict__ page_table, int table_width, int n_tiles, int n_heads, int n_kv,
                       float scale) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);              // [64][HD]
    bf16* Ks = Qs + QT * HD;                                   // [2][64][HD]
    bf16* Vs = Ks + 2 * kPage * HD;                            // [2][64][HD]
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    kv = fresh(kv);

    const int head = blockIdx.y;
    int b, q0;
    find_work_item(cu_seqlens, n_seqs, QT, n_tiles - 1 - (int)blockIdx.x, b, q0);   // long tiles (late rows of long prompts) first
    if (b < 0) return;
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
    const int s0 = start[b];
    const int rows = min(QT, q_len - q0);
    const int kvh = head / (n_heads / n_kv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kv_len = s0 + q_len;
    const int last_key = s0 + q0 + rows - 1;
    const int n_ktiles = last_key / kPage + 1;
    const int64_t page_elems = (int64_t)2 * n_kv * kPage * HD;

    auto tile_ptr = [&](int kt) {
        const int page = page_table[(int64_t)b * table_width + kt];
        return kv + page * page_elems + ((int64_t)kvh * kPage) * HD;
    };

    // query tile (rows past the end repeat the last valid row) and the first key/value page
    for (int i = tid; i < QT * CHUNKS; i += 128) {
        const int row = i / CHUNKS, c = i % CHUNKS;
        const int src_row = min(row, rows - 1);
        cp_async16(Qs + row * HD + swz(row, c) * 8, q + ((int64_t)(tok0 + q0 + src_row) * n_heads + head) * HD + c * 8, true);
    }
    {
        const bf16* kp = tile_ptr(0);
        load_tile(Ks, kp, kv_len);
        load_tile(Vs, kp + (int64_t)n_kv * kPage * HD, kv_len);
    }
    cp_async_commit();

    // per-thread rows: r_lo = 16 warp + lane / 4, r_hi = r_lo + 8
    const int r_lo = warp * 16 + (lane >> 2);
    const int pos_lo = s0 + q0 + min(r_lo, rows - 1), pos_hi = s0 + q0 + min(r_lo + 8, rows - 1);
    const float sl2 = scale * 1.4426950408889634f;              // scores in units of log2(e)

    uint32_t qf[KS][4];
    float o[ND][4];
#pragma unroll
    for (int d = 0; d < ND; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int kt = 0; kt < n_ktiles; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < n_ktiles) {                                // prefetch the next page into the other buffer
            const bf16* kp = tile_ptr(kt + 1);
            const int valid = kv_len - (kt + 1) * kPage;
            load_tile(Ks + (buf ^ 1) * kPage * HD, kp, valid);
            load_tile(Vs + (buf ^ 1) * kPage * HD, kp + (int64_t)n_kv * kPage * HD, valid);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kt == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qf[ks], Qs + row * HD + swz(row, 2 * ks + (lane >> 4)) * 8);
            }
        }
        const bf16* Kb = Ks + buf * kPage * HD;
        const bf16* Vb = Vs + buf * kPage * HD;

        // ---- S = Q K^T for 64 keys: 8 blocks of 8 keys ----
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int nb = 0; nb < 8; nb += 2) {
                uint32_t kf[4];
                const int key = 8 * (nb + (lane >> 4)) + (lane & 7);
                ldmatrix_x4(kf, Kb + key * HD + swz(key, 2 * ks + ((lane >> 3) & 1)) * 8);
                mma16816(s[nb], qf[ks], kf[0], kf[1]);
                mma16816(s[nb + 1], qf[ks], kf[2], kf[3]);
            }
        }
        // ---- mask, running maximum, probabilities ----
        const int key0 = kt * kPage + (lane & 3) * 2;
        const bool need_mask = kt * kPage + kPage - 1 > s0 + q0 + min(warp * 16, rows - 1);   // a key may lie after a row of this warp
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + nb * 8 + e;
                float a = s[nb][e] * sl2, c = s[nb][2 + e] * sl2;
                if (need_mask) {
                    if (key > pos_lo) a = -INFINITY;
                    if (key > pos_hi) c = -INFINITY;
                }
                s[nb][e] = a;
                s[nb][2 + e] = c;
                mx_lo = fmaxf(mx_lo, a);
                mx_hi = fmaxf(mx_hi, c);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);   // finite: key 0 is visible to every row
        const float c_lo = exp2f(m_lo - mn_lo), c_hi = exp2f(m_hi - mn_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nb][e] = exp2f(s[nb][e] - mn_lo);
                s[nb][2 + e] = exp2f(s[nb][2 + e] - mn_hi);
                sum_lo += s[nb][e];
                sum_hi += s[nb][2 + e];
            }
        }
        l_lo = l_lo * c_lo + sum_lo;                            // per-thread partial denominators; joined at the end
        l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
        for (int d = 0; d < ND; ++d) {
            o[d][0] *= c_lo; o[d][1] *= c_lo;
            o[d][2] *= c_hi; o[d][3] *= c_hi;
        }
        // ---- O += P V: 4 steps of 16 keys ----
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
            pf[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
            pf[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
            pf[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {
                uint32_t vf[4];
                const int key = 16 * j + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(vf, Vb + key * HD + swz(key, nd + (lane >> 4)) * 8);
                mma16816(o[nd], pf, vf[0], vf[1]);
                mma16816(o[nd + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();                                        // everyone is done with this buffer
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
    const int col = (lane & 3) * 2;
    if (r_lo < rows) {
        bf16* op = out + ((int64_t)(tok0 + q0 + r_lo) * n_heads + head) * HD + col;
#pragma unroll
        for (int d = 0; d < ND; ++d) *reinterpret_cast<uint32_t*>(op + d * 8) = pack_bf16(o[d][0] * i_lo, o[d][1] * i_lo);
    }
    if (r_lo + 8 < rows) {
        bf16* op = out + ((int64_t)(tok0 + q0 + r_lo + 8) * n_heads + head) * HD + col;
#pragma unroll
        for (int d = 0; d < ND; ++d) *reinterpret_cast<uint32_t*>(op + d * 8) = pack_bf16(o[d][2] * i_hi, o[d][3] * i_hi);
    }
}

}  // namespace promptmma
}  // namespace wick

using namespace wick;

WICK_API int wick_attn_prompt_mma_supported() { return promptmma::SUPPORTED ? 1 : 0; }

// Same arguments as wick_attn_prompt_bf16 (attn.cu).
WICK_API int wick_attn_prompt_mma_bf16(const void* q, const void* kv, void* out, int n_tiles, const int* cu_seqlens,
                                       int n_seqs, const int* start, const int* page_table,
                                       int table_width, int n_heads, int n_kv, float scale, void* s) {
    using namespace promptmma;
    WICK_REQUIRE(SUPPORTED, "attention (tensor cores): head_dim %d is beyond 128", HD);
    WICK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads over %d kv heads", n_heads, n_kv);
    WICK_REQUIRE(n_heads <= 65535, "attention: %d heads is beyond the grid limit", n_heads);
    if (n_tiles == 0) return 0;
    const size_t smem = (size_t)(QT + 4 * kPage) * HD * sizeof(bf16);
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        WICK_CUDA(cudaFuncSetAttribute(attn_prompt_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised = true;
    }
    WICK_CUDA(launch(attn_prompt_mma_kernel, dim3(n_tiles, n_heads), dim3(128), smem, (cudaStream_t)s, (const bf16*)q,
                     (const bf16*)kv, (bf16*)out, cu_seqlens, n_seqs, start, page_table, table_width, n_tiles,
                     n_heads, n_kv, scale));
    return check_launch("attn_prompt_mma");
}
