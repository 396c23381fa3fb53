// One kernel for the attention of a decode step with few sequences (bfloat16,
// head sizes 64 and 128, up to 8 query heads per kv head): what
// qk_norm_rope_append_kernel, attn_decode_mma_kernel and its merge kernel do in
// three launches.
//
// A cluster of S blocks (S <= 8, chosen by the host so that all blocks run at once)
// takes one (sequence, kv head); block r takes a contiguous run of the sequence's
// 128-position chunks.  Each block
//   * starts fetching its key and value pages at once (TMA, a ring of two stages
//     of two key pages and two value pages): the cache holds nothing that the
//     kernel before this one writes, so this overlaps that kernel's end;
//   * then waits for that kernel (the q/k/v projection), adds up its float32
//     partial sums for this kv head's query heads, norms and rotates them
//     (wick src/model.rs:475-480) and keeps them in shared memory as bfloat16;
//     the block whose run ends the sequence does the same for the new token's key
//     and value, writes them to the cache and patches them into the tile it has
//     fetched (the copy may have read that row before or after the write);
//   * runs its chunks like attn_decode_mma_kernel (scores with the keys on the
//     16-row side of mma.sync, one page per warp, two pairs of warps on alternate
//     chunks), each pair folding its chunks into a running maximum, sum and
//     accumulator in registers, in chunk order;
//   * merges its two pairs and stores the result into the shared memory of block 0
//     of the cluster, which merges the S blocks in block order and writes the
//     output rows.
// Every sum has a fixed order; there are no atomics.  Waits on copies are bounded.
// Formulas: wick src/model.rs:452-553.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace decodefused {

constexpr bool SUPPORTED = WICK_HD == 64 || WICK_HD == 128;
constexpr int HD = SUPPORTED ? WICK_HD : 64;           // other head sizes: the entry point refuses, the kernel is never launched
constexpr int PAGES = 2;
constexpr int CHUNK = PAGES * kPage;
constexpr int NH = 8;                                  // query heads of a kv head (the 8-wide side of the instruction)
constexpr int PANELS = HD / 64;
constexpr int PANEL_BYTES = kPage * 128;
constexpr int TILE_BYTES = PANELS * PANEL_BYTES;       // one page of keys (or values) of one kv head
constexpr int STAGE_BYTES = 2 * PAGES * TILE_BYTES;
constexpr int STAGES = 2;
constexpr int KS = HD / 16;
constexpr int GROUPS = 2;                              // pairs of compute warps (chunks alternate between them)
constexpr int CWARPS = GROUPS * PAGES;
constexpr int CTHREADS = CWARPS * 32;
constexpr int THREADS = CTHREADS + 32;                 // compute warps, then the producer warp
constexpr int MAX_CLUSTER = 8;
constexpr int MAX_SPLITS = 8;                          // partial sums of the projection that the kernel adds up
constexpr int PART_FLOATS = NH * HD + 2 * NH;          // a block's result: accumulators, maxima, sums
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + MAX_CLUSTER * PART_FLOATS * 4 + 1024;
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Byte offset, inside a page tile, of the 16-byte chunk `chunk` (8 elements) of row `row`.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * PANEL_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Store into block `rank` of the cluster, at the place `p` has in this block's shared memory.
__device__ __forceinline__ void st_remote(float* p, uint32_t rank, float v) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
// A load of something that a kernel still in flight when this one starts has written
// (the projection's partial sums, the rotation tables): never through the read-only
// path, and never moved above the wait for that kernel (which the compiler may do with
// an ordinary load through a const __restrict__ pointer).
__device__ __forceinline__ float ld_fresh(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
// 2^(a - b) for maxima that may be -inf (nothing seen yet): then the weight is 0.
__device__ __forceinline__ float weight(float a, float b) { return a == -INFINITY ? 0.f : exp2f(a - b); }

struct alignas(16) Shared {
    alignas(16) bf16 q[NH][HD];                        // normed, rotated query rows (rows beyond the group: zero)
    alignas(16) bf16 new_kv[2][HD];                    // the new token's key and value
    bf16 p[GROUPS][NH][CHUNK];
    float o[GROUPS][NH][HD];                           // a pair's second warp hands its part to the first; then each pair's result
    float m_w[GROUPS][PAGES][NH], l_w[GROUPS][PAGES][NH];
    float fin_m[GROUPS][NH], fin_l[GROUPS][NH];
    uint64_t full_k[STAGES], full_v[STAGES], empty[STAGES];
    int abort_flag, stop[GROUPS];
};

__global__ void __launch_bounds__(THREADS, 1)
attn_decode_fused_kernel(const __grid_constant__ CUtensorMap kv_map, const float* parts, int splits,
                         int64_t split_stride, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                         const float* cos_t, const float* sin_t, bf16* __restrict__ kv,
                         bf16* __restrict__ out, const int* __restrict__ kv_len_arr, const int* __restrict__ page_table,
                         int table_width, int n_heads, int n_kv, float scale, int write_kv, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ Shared sh;

    pdl_trigger();
    cluster_arrive();                                            // "this block runs": awaited before anyone stores into it
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = (int)cluster_size(), rank = (int)cluster_rank();
    const int cid = blockIdx.x / S;
    const int b = cid / n_kv, kvh = cid % n_kv;
    const int group = n_heads / n_kv;
    const int kv_len = kv_len_arr[b];                            // written by the host before the step, like the page table
    const int C = (kv_len + CHUNK - 1) / CHUNK;                  // chunks of the sequence
    const int per = (C + S - 1) / S;
    const int c_begin = min(C, rank * per), c_end = min(C, c_begin + per);
    const int my_chunks = c_end - c_begin;
    const bool owner = write_kv && c_end == C && my_chunks > 0;  // this block's run ends with the new token
    uint8_t* stages = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    if (tid == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sh.full_k[s], 1);
            mbar_init(&sh.full_v[s], 1);
            mbar_init(&sh.empty[s], PAGES);                      // one arrival per compute warp of the pair
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CWARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int n = 0; n < my_chunks; ++n) {
                const int s = n % STAGES;
                const uint32_t round = n / STAGES;
                if (!mbar_wait(&sh.empty[s], (round & 1) ^ 1, &sh.abort_flag, status, 8)) break;
                const int key_begin = (c_begin + n) * CHUNK;
                const int n_pages = min(PAGES, (kv_len - key_begin + kPage - 1) / kPage);
                uint8_t* st = stages + (size_t)s * STAGE_BYTES;
                int page[PAGES];
                for (int w = 0; w < n_pages; ++w) page[w] = page_table[(int64_t)b * table_width + key_begin / kPage + w];
                mbar_expect_tx(&sh.full_k[s], (uint32_t)(n_pages * TILE_BYTES));
                for (int w = 0; w < n_pages; ++w)
                    for (int pn = 0; pn < PANELS; ++pn)
                        tma_load_2d(&kv_map, &sh.full_k[s], st + w * TILE_BYTES + pn * PANEL_BYTES, pn * 64, ((page[w] * 2 + 0) * n_kv + kvh) * kPage);
                mbar_expect_tx(&sh.full_v[s], (uint32_t)(n_pages * TILE_BYTES));
                for (int w = 0; w < n_pages; ++w)
                    for (int pn = 0; pn < PANELS; ++pn)
                        tma_load_2d(&kv_map, &sh.full_v[s], st + (PAGES + w) * TILE_BYTES + pn * PANEL_BYTES, pn * 64, ((page[w] * 2 + 1) * n_kv + kvh) * kPage);
            }
        }
        __syncwarp();
        cluster_wait();
    } else {
        // ---------------- the new token's rows ----------------
        pdl_wait();                                              // the projection's partial sums
        const int half = HD / 2;
        const int row_width = (n_heads + 2 * n_kv) * HD;
        const float* row = parts + (int64_t)b * row_width;
        // One head (a query head of the group; in the owner block also the key and the
        // value) per warp and turn.  A lane holds elements lane, lane + 32, ... of a head:
        // both members of each rotated pair (i, i + HD / 2).  All turns' loads are issued
        // before the first is used.
        constexpr int EPL = HD / 32;                             // elements per lane
        constexpr int TURNS = (NH + 2 + CWARPS - 1) / CWARPS;
        const int n_rows = NH + (owner ? 2 : 0);
        float v[TURNS][EPL];
#pragma unroll
        for (int t = 0; t < TURNS; ++t) {
            const int h = warp + t * CWARPS;
            const bool is_q = h < NH, is_v = h == NH + 1;
            const bool used = h < n_rows && !(is_q && h >= group);
            const int64_t off = is_q ? (int64_t)(kvh * group + h) * HD : (int64_t)(n_heads + (is_v ? n_kv : 0) + kvh) * HD;
            float raw[MAX_SPLITS][EPL];                         // all loads first, then the sums in index order
#pragma unroll
            for (int sp = 0; sp < MAX_SPLITS; ++sp)
#pragma unroll
                for (int e = 0; e < EPL; ++e)
                    raw[sp][e] = (used && sp < splits) ? ld_fresh(row + sp * split_stride + off + lane + 32 * e) : 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                float x = raw[0][e];
#pragma unroll
                for (int sp = 1; sp < MAX_SPLITS; ++sp)
                    if (sp < splits) x += raw[sp][e];
                v[t][e] = x;
            }
        }
#pragma unroll
        for (int t = 0; t < TURNS; ++t) {
            const int h = warp + t * CWARPS;
            if (h >= n_rows) continue;
            const bool is_q = h < NH, is_v = h == NH + 1;
            bf16* dst = is_q ? sh.q[h] : sh.new_kv[is_v ? 1 : 0];
            const float* w = is_v ? nullptr : (is_q ? q_w : k_w);
            float sc = 1.f;
            if (w) {
                float ss = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) ss += v[t][e] * v[t][e];
                ss = warp_sum(ss);
                sc = 1.0f / sqrtf(ss / (float)HD + eps);
            }
#pragma unroll
            for (int e = 0; e < EPL / 2; ++e) {
                const int i = lane + 32 * e;                     // < HD / 2; its partner is i + HD / 2
                float x = v[t][e], y = v[t][e + EPL / 2];
                if (w) {
                    x = (x * sc) * w[i];
                    y = (y * sc) * w[i + half];
                }
                if (cos_t && !is_v) {
                    const float c = ld_fresh(cos_t + (int64_t)b * half + i), sn = ld_fresh(sin_t + (int64_t)b * half + i);
                    const float rx = x * c - y * sn, ry = y * c + x * sn;
                    x = rx;
                    y = ry;
                }
                dst[i] = __float2bfloat16_rn(x);
                dst[i + half] = __float2bfloat16_rn(y);
            }
        }
        asm volatile("bar.sync 3, %0;" ::"n"(CTHREADS) : "memory");
        // ---------------- chunks: GROUPS pairs of warps, one page per warp ----------------
        const float sl2 = scale * 1.4426950408889634f;
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;           // accumulator rows r0, r0 + 8; columns c0, c0 + 1
        const int grp = warp / PAGES;
        const int ctid = tid - grp * PAGES * 32;                 // 0..63 within the pair
        const int wp = warp % PAGES;                             // this warp's page of a chunk
        bf16 (*p_s)[CHUNK] = sh.p[grp];
        float (*o_s)[HD] = sh.o[grp];
        float (*m_w)[NH] = sh.m_w[grp];
        float (*l_w)[NH] = sh.l_w[grp];
        const int bar_id = 1 + grp;                              // named barrier of this pair
        // the pair's running result (kept by its first warp): maxima in units of log2 e
        float mr0 = -INFINITY, mr1 = -INFINITY, lr0 = 0.f, lr1 = 0.f;
        float acc[KS][4];
#pragma unroll
        for (int mb = 0; mb < KS; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;
        uint32_t qb[KS][2];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qb[ks][0] = *reinterpret_cast<const uint32_t*>(&sh.q[r0][16 * ks + c0]);
            qb[ks][1] = *reinterpret_cast<const uint32_t*>(&sh.q[r0][16 * ks + c0 + 8]);
        }
        for (int n = grp; n < my_chunks; n += GROUPS) {
            const int s = n % STAGES;
            const uint32_t round = n / STAGES;
            const int key_begin = (c_begin + n) * CHUNK;
            const int n_pages = min(PAGES, (kv_len - key_begin + kPage - 1) / kPage);
            const bool live = wp < n_pages;
            const int keys_here = live ? min(kPage, kv_len - key_begin - wp * kPage) : 0;
            // the new token's row of this warp's page, if it lies there and was computed here
            const int new_row = (owner && c_begin + n == C - 1 && (kv_len - 1 - key_begin) / kPage == wp) ? (kv_len - 1) % kPage : -1;
            uint8_t* st = stages + (size_t)s * STAGE_BYTES;
            const uint32_t k_base = smem_u32(st + wp * TILE_BYTES), v_base = smem_u32(st + (PAGES + wp) * TILE_BYTES);

            bool ok = mbar_wait(&sh.full_k[s], round & 1, &sh.abort_flag, status, 8);
            if (new_row >= 0 && ok) {
                if (lane < HD / 8)
                    *reinterpret_cast<uint4*>(st + wp * TILE_BYTES + tile_off(new_row, lane)) = reinterpret_cast<const uint4*>(sh.new_kv[0])[lane];
                __syncwarp();
            }
            // ---- scores S^T[key, head] of this warp's page ----
            float sc[4][4];
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (live && ok) {
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) {
                    sc[mb][0] = sc[mb][1] = sc[mb][2] = sc[mb][3] = 0.f;
                    const int row = 16 * mb + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        uint32_t a[4];
                        ldsm_x4(a, k_base + tile_off(row, 2 * ks + (lane >> 4)));
                        mma16816(sc[mb], a, qb[ks][0], qb[ks][1]);
                    }
                    const int ka = 16 * mb + r0, kb = ka + 8;
                    sc[mb][0] = ka < keys_here ? sc[mb][0] * sl2 : -INFINITY;
                    sc[mb][1] = ka < keys_here ? sc[mb][1] * sl2 : -INFINITY;
                    sc[mb][2] = kb < keys_here ? sc[mb][2] * sl2 : -INFINITY;
                    sc[mb][3] = kb < keys_here ? sc[mb][3] * sl2 : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(sc[mb][0], sc[mb][2]));
                    mx1 = fmaxf(mx1, fmaxf(sc[mb][1], sc[mb][3]));
                }
            }
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            }
            if (lane < 4) { m_w[wp][c0] = mx0; m_w[wp][c0 + 1] = mx1; }
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
            const float m0 = fmaxf(m_w[0][c0], m_w[1][c0]), m1 = fmaxf(m_w[0][c0 + 1], m_w[1][c0 + 1]);
            float l0 = 0.f, l1 = 0.f;
            if (live && ok) {
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) {
                    const float p0 = exp2f(sc[mb][0] - m0), p1 = exp2f(sc[mb][1] - m1);
                    const float p2 = exp2f(sc[mb][2] - m0), p3 = exp2f(sc[mb][3] - m1);
                    l0 += p0 + p2;
                    l1 += p1 + p3;
                    const int ka = wp * kPage + 16 * mb + r0;
                    p_s[c0][ka] = __float2bfloat16_rn(p0);
                    p_s[c0 + 1][ka] = __float2bfloat16_rn(p1);
                    p_s[c0][ka + 8] = __float2bfloat16_rn(p2);
                    p_s[c0 + 1][ka + 8] = __float2bfloat16_rn(p3);
                }
            }
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, o);
                l1 += __shfl_xor_sync(0xffffffffu, l1, o);
            }
            if (lane < 4) { l_w[wp][c0] = l0; l_w[wp][c0 + 1] = l1; }
            ok = mbar_wait(&sh.full_v[s], round & 1, &sh.abort_flag, status, 8) && ok;
            if (live && ok) {
                if (new_row >= 0 && lane < HD / 8)
                    *reinterpret_cast<uint4*>(st + (PAGES + wp) * TILE_BYTES + tile_off(new_row, lane)) = reinterpret_cast<const uint4*>(sh.new_kv[1])[lane];
                // Rows of the last page that hold no token yet may be anything: make them
                // zero, so that a zero weight times such a row stays zero.
                for (int i = lane; i < (kPage - keys_here) * (HD / 8); i += 32) {
                    const int row = keys_here + i / (HD / 8), chunk = i % (HD / 8);
                    *reinterpret_cast<uint4*>(st + (PAGES + wp) * TILE_BYTES + tile_off(row, chunk)) = make_uint4(0, 0, 0, 0);
                }
            }
            __syncwarp();
            // ---- O^T[dim, head] = V^T[dim, key] P[key, head] over this warp's keys ----
            float o[KS][4];
#pragma unroll
            for (int mb = 0; mb < KS; ++mb) o[mb][0] = o[mb][1] = o[mb][2] = o[mb][3] = 0.f;
            if (live && ok) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t pb0 = *reinterpret_cast<const uint32_t*>(&p_s[r0][wp * kPage + 16 * j + c0]);
                    const uint32_t pb1 = *reinterpret_cast<const uint32_t*>(&p_s[r0][wp * kPage + 16 * j + c0 + 8]);
                    const int key = 16 * j + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
                    for (int mb = 0; mb < KS; ++mb) {
                        uint32_t a[4];
                        ldsm_x4_trans(a, v_base + tile_off(key, 2 * mb + ((lane >> 3) & 1)));
                        mma16816(o[mb], a, pb0, pb1);
                    }
                }
            }
            // this warp has read all it needs of the stage
            __syncwarp();
            if (lane == 0) mbar_arrive_cta(&sh.empty[s]);
            // ---- the second warp hands its part to the first, which folds the chunk into the pair's result ----
            if (wp == 1) {
#pragma unroll
                for (int mb = 0; mb < KS; ++mb) {
                    o_s[c0][16 * mb + r0] = o[mb][0];
                    o_s[c0 + 1][16 * mb + r0] = o[mb][1];
                    o_s[c0][16 * mb + r0 + 8] = o[mb][2];
                    o_s[c0 + 1][16 * mb + r0 + 8] = o[mb][3];
                }
            }
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
            if (wp == 0 && ok) {
                const float n0 = fmaxf(mr0, m0), n1 = fmaxf(mr1, m1);
                const float a0 = weight(mr0, n0), b0 = weight(m0, n0), a1 = weight(mr1, n1), b1 = weight(m1, n1);
#pragma unroll
                for (int mb = 0; mb < KS; ++mb) {
                    const int d = 16 * mb + r0;
                    acc[mb][0] = acc[mb][0] * a0 + (o[mb][0] + o_s[c0][d]) * b0;
                    acc[mb][2] = acc[mb][2] * a0 + (o[mb][2] + o_s[c0][d + 8]) * b0;
                    acc[mb][1] = acc[mb][1] * a1 + (o[mb][1] + o_s[c0 + 1][d]) * b1;
                    acc[mb][3] = acc[mb][3] * a1 + (o[mb][3] + o_s[c0 + 1][d + 8]) * b1;
                }
                lr0 = lr0 * a0 + (l_w[0][c0] + l_w[1][c0]) * b0;
                lr1 = lr1 * a1 + (l_w[0][c0 + 1] + l_w[1][c0 + 1]) * b1;
                mr0 = n0;
                mr1 = n1;
            }
            if (ctid == 0) sh.stop[grp] = sh.abort_flag;                    // one decision for both warps
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");     // o_s, m_w, l_w, p_s are free again
            if (sh.stop[grp]) break;
        }
        if (owner) {
            // into the cache, for the steps to come
            const int pos = kv_len - 1;
            const int page = page_table[(int64_t)b * table_width + pos / kPage];
            for (int i = tid; i < 2 * (HD / 8); i += CTHREADS) {
                const int is_v = i / (HD / 8), chunk = i % (HD / 8);
                bf16* dst = kv + ((((int64_t)page * 2 + is_v) * n_kv + kvh) * kPage + (pos % kPage)) * HD;
                reinterpret_cast<uint4*>(dst)[chunk] = reinterpret_cast<const uint4*>(sh.new_kv[is_v])[chunk];
            }
        }
        // ---- each pair's result, then the block's ----
        if (wp == 0) {
#pragma unroll
            for (int mb = 0; mb < KS; ++mb) {
                o_s[c0][16 * mb + r0] = acc[mb][0];
                o_s[c0 + 1][16 * mb + r0] = acc[mb][1];
                o_s[c0][16 * mb + r0 + 8] = acc[mb][2];
                o_s[c0 + 1][16 * mb + r0 + 8] = acc[mb][3];
            }
            if (lane < 4) {
                sh.fin_m[grp][c0] = mr0;
                sh.fin_m[grp][c0 + 1] = mr1;
                sh.fin_l[grp][c0] = lr0;
                sh.fin_l[grp][c0 + 1] = lr1;
            }
        }
        asm volatile("bar.sync 3, %0;" ::"n"(CTHREADS) : "memory");
        // the block's result goes to block 0 of the cluster (stores into its shared memory, once it runs)
        cluster_wait();
        float* gather = reinterpret_cast<float*>(stages + (size_t)STAGES * STAGE_BYTES) + (size_t)rank * PART_FLOATS;
        for (int idx = tid; idx < NH * HD; idx += CTHREADS) {
            const int h = idx / HD, d = idx % HD;
            const float ma = sh.fin_m[0][h], mb = sh.fin_m[1][h];
            const float mm = fmaxf(ma, mb);
            const float wa = weight(ma, mm), wb = weight(mb, mm);
            st_remote(gather + idx, 0, sh.o[0][h][d] * wa + sh.o[1][h][d] * wb);
            if (d == 0) {
                st_remote(gather + NH * HD + h, 0, mm);
                st_remote(gather + NH * HD + NH + h, 0, sh.fin_l[0][h] * wa + sh.fin_l[1][h] * wb);
            }
        }
    }

    // ---------------- the cluster's blocks, in block order ----------------
    __syncthreads();
    cluster_arrive();
    cluster_wait();                                            // every block's result has arrived in block 0
    if (rank == 0 && !sh.abort_flag) {
        const float* all = reinterpret_cast<const float*>(stages + (size_t)STAGES * STAGE_BYTES);
        for (int idx = tid; idx < group * HD; idx += THREADS) {
            const int h = idx / HD, d = idx % HD;
            float pm[MAX_CLUSTER], po[MAX_CLUSTER], pl[MAX_CLUSTER];
#pragma unroll
            for (int r = 0; r < MAX_CLUSTER; ++r) {
                const bool in = r < S;
                pm[r] = in ? all[r * PART_FLOATS + NH * HD + h] : -INFINITY;
                po[r] = in ? all[r * PART_FLOATS + idx] : 0.f;
                pl[r] = in ? all[r * PART_FLOATS + NH * HD + NH + h] : 0.f;
            }
            float mm = -INFINITY;
#pragma unroll
            for (int r = 0; r < MAX_CLUSTER; ++r) mm = fmaxf(mm, pm[r]);
            float o = 0.f, l = 0.f;
#pragma unroll
            for (int r = 0; r < MAX_CLUSTER; ++r) {
                const float w = weight(pm[r], mm);
                o = fmaf(po[r], w, o);
                l = fmaf(pl[r], w, l);
            }
            out[((int64_t)b * n_heads + kvh * group + h) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        }
    }
    if (sh.abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000); // copies in flight land before the block leaves
    }
}

}  // namespace decodefused
}  // namespace wick

using namespace wick;

// Whether the fused kernel takes this problem: head size 64 or 128, at most 8 query
// heads per kv head, and few enough (sequence, kv head) pairs for all blocks to run at once.
WICK_API int wick_attn_decode_fused_supported(int n_seqs, int n_heads, int n_kv) {
    using namespace decodefused;
    if (!SUPPORTED || n_kv <= 0 || n_heads % n_kv != 0 || n_heads / n_kv > NH) return 0;
    return (long long)n_seqs * n_kv <= 148 ? 1 : 0;
}

// parts: float32 [splits, n_seqs, (n_heads + 2 n_kv) HD] partial sums of the q/k/v projection;
// q_w, k_w: per-head norm weights [HD] or null; cos_t, sin_t: [n_seqs, HD / 2] or null;
// kv: one schedule entry's cache [kv_pages, 2, n_kv, 64, HD] bfloat16; kv_len: positions per
// sequence including the new token; out: bfloat16 [n_seqs, n_heads, HD]; status: device int
// (code 8 if a block gave up waiting for its copies).
WICK_API int wick_attn_decode_fused_bf16(const float* parts, int splits, int n_seqs, const float* q_w, const float* k_w,
                                         float eps, const float* cos_t, const float* sin_t, void* kv, long long kv_pages,
                                         void* out, const int* kv_len, int max_kv_len, const int* page_table,
                                         int table_width, int n_heads, int n_kv, float scale, int write_kv, int* status,
                                         void* s) {
    using namespace decodefused;
    WICK_REQUIRE(SUPPORTED, "attention decode (fused): head_dim %d is not 64 or 128", (int)WICK_HD);
    WICK_REQUIRE(wick_attn_decode_fused_supported(n_seqs, n_heads, n_kv), "attention decode (fused): %d sequences, %d heads over %d kv heads is beyond this kernel", n_seqs, n_heads, n_kv);
    WICK_REQUIRE(splits >= 1 && splits <= MAX_SPLITS, "attention decode (fused): %d partial sums, at most %d", splits, MAX_SPLITS);
    if (n_seqs == 0) return 0;
    CUtensorMap map;
    if (int e = make_bf16_map(&map, kv, kv_pages * 2 * n_kv * kPage, HD, kPage, "attention decode (fused)")) return e;
    const int pairs = n_seqs * n_kv;
    const int chunks = ceil_div(max_kv_len > 0 ? max_kv_len : 1, CHUNK);
    int S = 148 / pairs;
    if (S > MAX_CLUSTER) S = MAX_CLUSTER;
    if (S > chunks) S = chunks;
    if (S < 1) S = 1;
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        raised = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pairs * S);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = (cudaStream_t)s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    const int64_t split_stride = (int64_t)n_seqs * (n_heads + 2 * n_kv) * HD;
    WICK_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel, map, parts, splits, split_stride, q_w, k_w, eps, cos_t, sin_t,
                                 (bf16*)kv, (bf16*)out, kv_len, page_table, table_width, n_heads, n_kv, scale, write_kv, status));
    return check_launch("attn_decode_fused");
}
