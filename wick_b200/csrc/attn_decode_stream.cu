// Decode attention of a step with many sequences in one kernel (bfloat16, head
// sizes 64 and 128, up to 8 query heads per kv head): what
// qk_norm_rope_append_kernel, attn_decode_mma_kernel and its merge kernel do in
// three launches, for more (sequence, kv head) jobs than there are SMs.  (Up to
// one job per SM, attn_decode_fused_kernel spreads a job over a cluster instead.)
//
// Persistent blocks, one per SM; block i takes jobs i, i + blocks, ...  A block has
// two pairs of warps that work independently: the pairs take the block's jobs in
// turn, and a pair runs a whole job:
//   * it adds up the projection's float32 partial sums for the job's query heads
//     and for the new token's key and value, norms and rotates them (wick
//     src/model.rs:475-480), keeps them in shared memory as bfloat16;
//   * it walks over the sequence's 128-position chunks (scores with the keys on the
//     16-row side of mma.sync, one page per warp), folding each into a running
//     maximum, sum and accumulator in registers, in chunk order; the new token's
//     key and value are patched into the last chunk's tile (the copy may have read
//     that row before or after it is written) and written to the cache;
//   * it divides by the sum and writes the output rows: nothing to merge.
// A producer warp feeds both pairs through one ring of three stages (TMA, two key
// pages and two value pages each): item 2 k + g of the ring is chunk k of pair g's
// jobs, so both sides know an item's stage without talking; when one pair has run
// out of chunks its items are skipped.  Barriers exist per (stage, pair): a pair
// meets a stage every sixth item, and with a barrier of its own it sees every
// phase of it (a barrier shared by both pairs would be waited for two phases
// apart, which a parity cannot tell from none: that held only while copies
// completed in the order of their issue, and a launch of this kernel failed).
// While one pair prepares a job's query rows (a chain of loads), the other
// computes, and the copies of the chunks after next are in flight all the time.
// Every sum has a fixed order; there are no atomics.  Waits on copies are bounded.
// Formulas: wick src/model.rs:452-553.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace decodestream {

constexpr bool SUPPORTED = WICK_HD == 64 || WICK_HD == 128;
constexpr int HD = SUPPORTED ? WICK_HD : 64;           // other head sizes: the entry point refuses, the kernel is never launched
constexpr int PAGES = 2;
constexpr int CHUNK = PAGES * kPage;
constexpr int NH = 8;                                  // query heads of a kv head (the 8-wide side of the instruction)
constexpr int PANELS = HD / 64;
constexpr int PANEL_BYTES = kPage * 128;
constexpr int TILE_BYTES = PANELS * PANEL_BYTES;       // one page of keys (or values) of one kv head
constexpr int STAGE_BYTES = 2 * PAGES * TILE_BYTES;
constexpr int STAGES = 3;
constexpr int KS = HD / 16;
constexpr int GROUPS = 2;                              // pairs of compute warps (jobs alternate between them)
static_assert(STAGES == 3 && GROUPS == 2, "the barriers count on a pair meeting a stage every STAGES * GROUPS items");
constexpr int CWARPS = GROUPS * PAGES;
constexpr int GTHREADS = PAGES * 32;                   // threads of a pair
constexpr int THREADS = CWARPS * 32 + 32;              // compute warps, then the producer warp
constexpr int MAX_SPLITS = 8;                          // partial sums of the projection that the kernel adds up
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
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
    alignas(16) bf16 q[GROUPS][NH][HD];                // normed, rotated query rows (rows beyond the group: zero)
    alignas(16) bf16 new_kv[GROUPS][2][HD];            // the new token's key and value
    bf16 p[GROUPS][NH][CHUNK];
    float o[GROUPS][NH][HD];                           // a pair's second warp hands its part to the first; then the job's result
    float m_w[GROUPS][PAGES][NH], l_w[GROUPS][PAGES][NH];
    uint64_t full_k[STAGES][GROUPS], full_v[STAGES][GROUPS], empty[STAGES][GROUPS];
    int abort_flag, stop[GROUPS];
};

__global__ void __launch_bounds__(THREADS, 1)
attn_decode_stream_kernel(const __grid_constant__ CUtensorMap kv_map, const float* parts, int splits,
                          int64_t split_stride, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                          const float* cos_t, const float* sin_t, bf16* __restrict__ kv,
                          bf16* __restrict__ out, const int* __restrict__ kv_len_arr, const int* __restrict__ page_table,
                          int table_width, int n_jobs, int n_heads, int n_kv, float scale, int write_kv, int kv_pages, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ Shared sh;

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = n_heads / n_kv;
    uint8_t* stages = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // pair g's t-th job
    auto job_of = [&](int g, int t) { return (int)blockIdx.x + (2 * t + g) * (int)gridDim.x; };

    if (tid == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < STAGES; ++s)
            for (int g = 0; g < GROUPS; ++g) {
                mbar_init(&sh.full_k[s][g], 1);
                mbar_init(&sh.full_v[s][g], 1);
                mbar_init(&sh.empty[s][g], PAGES);               // one arrival per compute warp of the pair
            }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CWARPS) {
        // ---------------- producer ----------------
        // The cache holds nothing that the kernel before this one writes: the copies start at once.
        if (lane == 0) {
            int turn[GROUPS], chunk[GROUPS], chunks[GROUPS], b_of[GROUPS], kvh_of[GROUPS], len_of[GROUPS];
            auto open_job = [&](int g) {
                const int job = job_of(g, turn[g]);
                chunks[g] = 0;
                if (job < n_jobs) {
                    b_of[g] = job / n_kv;
                    kvh_of[g] = job % n_kv;
                    len_of[g] = kv_len_arr[b_of[g]];             // written by the host before the step, like the page table
                    chunks[g] = (len_of[g] + CHUNK - 1) / CHUNK;
                }
                chunk[g] = 0;
            };
            for (int g = 0; g < GROUPS; ++g) { turn[g] = 0; open_job(g); }
            int held_by[STAGES], held_parity[STAGES];            // the pair whose chunk a stage holds, and the phase that frees it
            for (int s = 0; s < STAGES; ++s) held_by[s] = -1;
            for (uint32_t n = 0; chunks[0] > 0 || chunks[1] > 0; ++n) {
                const int g = (int)(n % GROUPS), s = (int)(n % STAGES);
                if (chunks[g] == 0) continue;                    // this pair has no chunks left: nothing goes into the stage
                if (held_by[s] >= 0 && !mbar_wait(&sh.empty[s][held_by[s]], (uint32_t)held_parity[s], &sh.abort_flag, status, 8)) break;
                held_by[s] = g;
                held_parity[s] = (int)((n / (STAGES * GROUPS)) & 1);
                const int b = b_of[g], kvh = kvh_of[g], kv_len = len_of[g];
                const int key_begin = chunk[g] * CHUNK;
                const int n_pages = min(PAGES, (kv_len - key_begin + kPage - 1) / kPage);
                uint8_t* st = stages + (size_t)s * STAGE_BYTES;
                int page[PAGES];
                bool bad = key_begin / kPage + n_pages > table_width || n_pages < 1;
                for (int w = 0; w < n_pages && !bad; ++w) {
                    page[w] = page_table[(int64_t)b * table_width + key_begin / kPage + w];
                    bad = page[w] < 0 || page[w] >= kv_pages;
                }
                if (bad) {                                       // a page outside the cache: give up, say so
                    *(volatile int*)&sh.abort_flag = 1;
                    atomicCAS(status, 0, 10);
                    break;
                }
                mbar_expect_tx(&sh.full_k[s][g], (uint32_t)(n_pages * TILE_BYTES));
                for (int w = 0; w < n_pages; ++w)
                    for (int pn = 0; pn < PANELS; ++pn)
                        tma_load_2d(&kv_map, &sh.full_k[s][g], st + w * TILE_BYTES + pn * PANEL_BYTES, pn * 64, ((page[w] * 2 + 0) * n_kv + kvh) * kPage);
                mbar_expect_tx(&sh.full_v[s][g], (uint32_t)(n_pages * TILE_BYTES));
                for (int w = 0; w < n_pages; ++w)
                    for (int pn = 0; pn < PANELS; ++pn)
                        tma_load_2d(&kv_map, &sh.full_v[s][g], st + (PAGES + w) * TILE_BYTES + pn * PANEL_BYTES, pn * 64, ((page[w] * 2 + 1) * n_kv + kvh) * kPage);
                if (++chunk[g] == chunks[g]) {
                    ++turn[g];
                    open_job(g);
                }
            }
        }
        __syncwarp();
    } else {
        const int grp = warp / PAGES;
        const int wp = warp % PAGES;                             // this warp's page of a chunk
        const int ctid = tid - grp * GTHREADS;                   // 0..63 within the pair
        const int bar_id = 1 + grp;                              // named barrier of this pair
        bf16 (*q_s)[HD] = sh.q[grp];
        bf16 (*nkv_s)[HD] = sh.new_kv[grp];
        bf16 (*p_s)[CHUNK] = sh.p[grp];
        float (*o_s)[HD] = sh.o[grp];
        float (*m_w)[NH] = sh.m_w[grp];
        float (*l_w)[NH] = sh.l_w[grp];
        const float sl2 = scale * 1.4426950408889634f;
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;           // accumulator rows r0, r0 + 8; columns c0, c0 + 1
        const int half = HD / 2;
        const int row_width = (n_heads + 2 * n_kv) * HD;
        pdl_wait();                                              // the projection's partial sums
        uint32_t k_item = 0;                                     // chunks of this pair so far: chunk k is item 2 k + grp of the ring
        bool stop = false;
        for (int t = 0; !stop; ++t) {
            const int job = job_of(grp, t);
            if (job >= n_jobs) break;
            const int b = job / n_kv, kvh = job % n_kv;
            const int kv_len = kv_len_arr[b];
            const int C = (kv_len + CHUNK - 1) / CHUNK;
            // ---------------- the new token's rows ----------------
            // One head (a query head of the group, the key, the value) per warp and turn.  A lane
            // holds elements lane, lane + 32, ... of a head: both members of each rotated pair
            // (i, i + HD / 2).  A turn's loads are all issued before the first is used.
            {
                const float* row = parts + (int64_t)b * row_width;
                constexpr int EPL = HD / 32;                     // elements per lane
                constexpr int TURNS = (NH + 2 + PAGES - 1) / PAGES;
                const int n_rows = NH + (write_kv ? 2 : 0);
#pragma unroll 1
                for (int u = 0; u < TURNS; ++u) {
                    const int h = wp + u * PAGES;
                    if (h >= n_rows) break;
                    const bool is_q = h < NH, is_v = h == NH + 1;
                    const bool used = !(is_q && h >= group);
                    const int64_t off = is_q ? (int64_t)(kvh * group + h) * HD : (int64_t)(n_heads + (is_v ? n_kv : 0) + kvh) * HD;
                    float raw[MAX_SPLITS][EPL];                  // all loads first, then the sums in index order
#pragma unroll
                    for (int sp = 0; sp < MAX_SPLITS; ++sp)
#pragma unroll
                        for (int e = 0; e < EPL; ++e)
                            raw[sp][e] = (used && sp < splits) ? ld_fresh(row + sp * split_stride + off + lane + 32 * e) : 0.f;
                    float cs[EPL / 2], sn[EPL / 2];
                    const bool rotate = cos_t && !is_v;
#pragma unroll
                    for (int e = 0; e < EPL / 2; ++e) {
                        cs[e] = rotate ? ld_fresh(cos_t + (int64_t)b * half + lane + 32 * e) : 1.f;
                        sn[e] = rotate ? ld_fresh(sin_t + (int64_t)b * half + lane + 32 * e) : 0.f;
                    }
                    float v[EPL];
#pragma unroll
                    for (int e = 0; e < EPL; ++e) {
                        float x = raw[0][e];
#pragma unroll
                        for (int sp = 1; sp < MAX_SPLITS; ++sp)
                            if (sp < splits) x += raw[sp][e];
                        v[e] = x;
                    }
                    bf16* dst = is_q ? q_s[h] : nkv_s[is_v ? 1 : 0];
                    const float* w = is_v ? nullptr : (is_q ? q_w : k_w);
                    float sc = 1.f;
                    if (w) {
                        float ss = 0.f;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) ss += v[e] * v[e];
                        ss = warp_sum(ss);
                        sc = 1.0f / sqrtf(ss / (float)HD + eps);
                    }
#pragma unroll
                    for (int e = 0; e < EPL / 2; ++e) {
                        const int i = lane + 32 * e;             // < HD / 2; its partner is i + HD / 2
                        float x = v[e], y = v[e + EPL / 2];
                        if (w) {
                            x = (x * sc) * w[i];
                            y = (y * sc) * w[i + half];
                        }
                        if (rotate) {
                            const float rx = x * cs[e] - y * sn[e], ry = y * cs[e] + x * sn[e];
                            x = rx;
                            y = ry;
                        }
                        dst[i] = __float2bfloat16_rn(x);
                        dst[i + half] = __float2bfloat16_rn(y);
                    }
                }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(GTHREADS) : "memory");
            // ---------------- the job's chunks, one page per warp ----------------
            // the running result (kept by the pair's first warp): maxima in units of log2 e
            float mr0 = -INFINITY, mr1 = -INFINITY, lr0 = 0.f, lr1 = 0.f;
            float acc[KS][4];
#pragma unroll
            for (int mb = 0; mb < KS; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;
            uint32_t qb[KS][2];
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                qb[ks][0] = *reinterpret_cast<const uint32_t*>(&q_s[r0][16 * ks + c0]);
                qb[ks][1] = *reinterpret_cast<const uint32_t*>(&q_s[r0][16 * ks + c0 + 8]);
            }
            for (int n = 0; n < C; ++n, ++k_item) {
                const uint32_t item = GROUPS * k_item + grp;
                const int s = (int)(item % STAGES);
                const uint32_t visit = item / (STAGES * GROUPS);   // this pair's visits to this stage so far
                const int key_begin = n * CHUNK;
                const int n_pages = min(PAGES, (kv_len - key_begin + kPage - 1) / kPage);
                const bool live = wp < n_pages;
                const int keys_here = live ? min(kPage, kv_len - key_begin - wp * kPage) : 0;
                // the new token's row of this warp's page, if it lies there
                const int new_row = (write_kv && n == C - 1 && (kv_len - 1 - key_begin) / kPage == wp) ? (kv_len - 1) % kPage : -1;
                uint8_t* st = stages + (size_t)s * STAGE_BYTES;
                const uint32_t k_base = smem_u32(st + wp * TILE_BYTES), v_base = smem_u32(st + (PAGES + wp) * TILE_BYTES);

                bool ok = mbar_wait(&sh.full_k[s][grp], visit & 1, &sh.abort_flag, status, 8);
                if (new_row >= 0 && ok) {
                    if (lane < HD / 8)
                        *reinterpret_cast<uint4*>(st + wp * TILE_BYTES + tile_off(new_row, lane)) = reinterpret_cast<const uint4*>(nkv_s[0])[lane];
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
                ok = mbar_wait(&sh.full_v[s][grp], visit & 1, &sh.abort_flag, status, 8) && ok;
                if (live && ok) {
                    if (new_row >= 0 && lane < HD / 8)
                        *reinterpret_cast<uint4*>(st + (PAGES + wp) * TILE_BYTES + tile_off(new_row, lane)) = reinterpret_cast<const uint4*>(nkv_s[1])[lane];
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
                if (lane == 0) mbar_arrive_cta(&sh.empty[s][grp]);
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
if (ctid == 0) sh.stop[grp] = sh.abort_flag;                // one decision for both warps
                asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(GTHREADS) : "memory");   // o_s, m_w, l_w, p_s are free again
                if (sh.stop[grp]) { stop = true; break; }
            }
            if (stop) break;
            if (write_kv) {
                // into the cache, for the steps to come
                const int pos = kv_len - 1;
                const int page = page_table[(int64_t)b * table_width + pos / kPage];
                if (page < 0 || page >= kv_pages || pos / kPage >= table_width) {
                    *(volatile int*)&sh.abort_flag = 1;
                    atomicCAS(status, 0, 10);
                } else
                for (int i = ctid; i < 2 * (HD / 8); i += GTHREADS) {
                    const int is_v = i / (HD / 8), chunk = i % (HD / 8);
                    bf16* dst = kv + ((((int64_t)page * 2 + is_v) * n_kv + kvh) * kPage + (pos % kPage)) * HD;
                    reinterpret_cast<uint4*>(dst)[chunk] = reinterpret_cast<const uint4*>(nkv_s[is_v])[chunk];
                }
            }
            // ---- the job's result: divided by the sum, through shared memory, as whole rows ----
            if (wp == 0) {
                const float i0 = lr0 > 0.f ? 1.0f / lr0 : 0.f, i1 = lr1 > 0.f ? 1.0f / lr1 : 0.f;
#pragma unroll
                for (int mb = 0; mb < KS; ++mb) {
                    o_s[c0][16 * mb + r0] = acc[mb][0] * i0;
                    o_s[c0 + 1][16 * mb + r0] = acc[mb][1] * i1;
                    o_s[c0][16 * mb + r0 + 8] = acc[mb][2] * i0;
                    o_s[c0 + 1][16 * mb + r0 + 8] = acc[mb][3] * i1;
                }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(GTHREADS) : "memory");
            for (int idx = ctid * 2; idx < group * HD; idx += GTHREADS * 2) {
                const int h = idx / HD, d = idx % HD;
                *reinterpret_cast<__nv_bfloat162*>(out + ((int64_t)b * n_heads + kvh * group + h) * HD + d) =
                    __floats2bfloat162_rn(o_s[h][d], o_s[h][d + 1]);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(GTHREADS) : "memory");   // q_s, o_s are free for the next job
        }
    }

    __syncthreads();
    if (sh.abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000); // copies in flight land before the block leaves
    }
}

}  // namespace decodestream
}  // namespace wick

using namespace wick;

// Whether the kernel takes this problem: head size 64 or 128, at most 8 query heads per kv head.
WICK_API int wick_attn_decode_stream_supported(int n_seqs, int n_heads, int n_kv) {
    using namespace decodestream;
    if (!SUPPORTED || n_seqs < 0 || n_kv <= 0 || n_heads % n_kv != 0 || n_heads / n_kv > NH) return 0;
    return 1;
}

// The arguments of wick_attn_decode_fused_bf16 (attn_decode_fused.cu), for any number of sequences.
WICK_API int wick_attn_decode_stream_bf16(const float* parts, int splits, int n_seqs, const float* q_w, const float* k_w,
                                          float eps, const float* cos_t, const float* sin_t, void* kv, long long kv_pages,
                                          void* out, const int* kv_len, int max_kv_len, const int* page_table,
                                          int table_width, int n_heads, int n_kv, float scale, int write_kv, int* status,
                                          void* s) {
    using namespace decodestream;
    (void)max_kv_len;
    WICK_REQUIRE(SUPPORTED, "attention decode (stream): head_dim %d is not 64 or 128", (int)WICK_HD);
    WICK_REQUIRE(wick_attn_decode_stream_supported(n_seqs, n_heads, n_kv), "attention decode (stream): %d heads over %d kv heads is beyond this kernel", n_heads, n_kv);
    WICK_REQUIRE(splits >= 1 && splits <= MAX_SPLITS, "attention decode (stream): %d partial sums, at most %d", splits, MAX_SPLITS);
    WICK_REQUIRE((long long)n_seqs * n_kv < (1ll << 30), "attention decode (stream): too many sequences");
    if (n_seqs == 0) return 0;
    CUtensorMap map;
    if (int e = make_bf16_map(&map, kv, kv_pages * 2 * n_kv * kPage, HD, kPage, "attention decode (stream)")) return e;
    const int jobs = n_seqs * n_kv;
    const int blocks = jobs < 148 ? jobs : 148;
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        raised = true;
    }
    const int64_t split_stride = (int64_t)n_seqs * (n_heads + 2 * n_kv) * HD;
    WICK_CUDA(launch(attn_decode_stream_kernel, dim3(blocks), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)s, map, parts, splits,
                     split_stride, q_w, k_w, eps, cos_t, sin_t, (bf16*)kv, (bf16*)out, kv_len, page_table, table_width, jobs,
                     n_heads, n_kv, scale, write_kv, (int)kv_pages, status));
    return check_launch("attn_decode_stream");
}
