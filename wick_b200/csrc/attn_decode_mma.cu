// Decode attention on the tensor cores (bfloat16, head sizes that are multiples
// of 64): one new token per sequence over the paged cache.
//
// A work item is (sequence, kv head, split of 128 positions, group of up to 8
// query heads).  Persistent blocks (one per SM) take items round-robin and run
// them through a ring of three shared-memory stages:
//   * a producer warp fetches an item's two key pages, two value pages (TMA,
//     64 x 64 boxes, 128-byte swizzle) and its query rows (bulk copy) while the
//     compute warps are still busy with earlier items, so that the memory
//     system always has several items in flight per SM;
//   * scores: S^T[keys, heads] = K[keys, dims] Q^T as mma.sync m16n8k16 with the
//     keys on the 16-row side (no padding rows), one page per compute warp;
//   * softmax statistics per head over the item's keys in float32; the
//     probabilities go through shared memory as bfloat16;
//   * values: O^T[dims, heads] = V^T[dims, keys] P[keys, heads] (ldmatrix.trans);
//   * each item writes its unnormalised partial result with its maximum and
//     denominator; a second kernel merges the splits of a sequence in index order.
// Two pairs of compute warps work on alternate items, so that one pair's waits
// (barriers, stores) are covered by the other's arithmetic.
// Formulas: wick src/model.rs:520-553.  The plain forms of this computation are
// attn_decode_fast_kernel (attn_decode.cu) and attn_decode_kernel (attn.cu).
#include "common.cuh"
#include "sm100.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace decodemma {

constexpr int HD = WICK_HD;
constexpr bool SUPPORTED = HD % 64 == 0 && HD <= 128;
constexpr int PAGES = 2;
constexpr int SPLIT = PAGES * kPage;
constexpr int NH = 8;                                  // query heads per item (the 8-wide side of the instruction)
constexpr int PANELS = SUPPORTED ? HD / 64 : 1;        // 64-column panels of a row (one TMA box each)
constexpr int PANEL_BYTES = kPage * 128;
constexpr int TILE_BYTES = PANELS * PANEL_BYTES;       // one page of keys (or values) of one kv head
constexpr int Q_BYTES = NH * HD * 2;
constexpr int STAGE_BYTES = 2 * PAGES * TILE_BYTES + 2048;   // keys, values, query rows (8 x 128 x 2 bytes at most)
static_assert(Q_BYTES <= 2048 || !SUPPORTED, "the query rows of an item fit the space kept for them");
constexpr int STAGES = 3;
constexpr int KS = HD / 16;
constexpr int GROUPS = 2;                              // independent pairs of compute warps (items alternate between them)
static_assert(STAGES == 3 && GROUPS == 2, "the barriers count on a pair meeting a stage every STAGES * GROUPS items");
constexpr int CWARPS = GROUPS * PAGES;
constexpr int THREADS = (CWARPS + 1) * 32;             // compute warps (one page each), then the producer warp
constexpr int MAX_SEQS = 512;
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

struct Item { int b, kvh, split, h0, nh, kv_len; };

__global__ void __launch_bounds__(THREADS, 1)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q, bf16* __restrict__ out,
                       float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ kv_len_arr, const int* __restrict__ page_table, int table_width,
                       int n_seqs, int n_heads, int n_kv, int max_splits, float scale, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(16) bf16 p_all[GROUPS][NH][SPLIT];
    __shared__ float o_all[GROUPS][NH][HD];              // the second warp's part of the output
    __shared__ float m_all[GROUPS][PAGES][NH], l_all[GROUPS][PAGES][NH];
    __shared__ int cum[MAX_SEQS + 1];                    // items before each sequence
    __shared__ int kvl[MAX_SEQS];                        // cached positions of each sequence
    // Barriers per (stage, pair of warps).  Item n goes to stage n % 3 and to pair n % 2, so a pair
    // comes back to a stage every sixth item: with one barrier per stage for both pairs, a pair's
    // wait would lie two phases after its last one, which a parity cannot tell from none, and the
    // wait would hold only as long as copies complete in the order they were issued.  With a
    // barrier of its own, every waiter sees every phase: visit n / 6 has parity (n / 6) & 1.
    __shared__ uint64_t full_k[STAGES][GROUPS], full_v[STAGES][GROUPS], empty[STAGES][GROUPS];
    __shared__ int abort_flag, stop_s[GROUPS];

    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = n_heads / n_kv;
    const int n_pass = (group + NH - 1) / NH;
    uint8_t* stages = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    // items before each sequence: sequence b has n_kv * ceil(kv_len / 128) * n_pass of them
    if (warp == 0) {
        int carry = 0;
        for (int b0 = 0; b0 < n_seqs; b0 += 32) {
            const int b = b0 + lane;
            const int len = b < n_seqs ? kv_len_arr[b] : 0;
            if (b < n_seqs) kvl[b] = len;
            int n = b < n_seqs ? n_kv * ((len + SPLIT - 1) / SPLIT) * n_pass : 0;
            int incl = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (b < n_seqs) cum[b] = carry + incl - n;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) cum[n_seqs] = carry;
    }
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s)
            for (int g = 0; g < GROUPS; ++g) {
                mbar_init(&full_k[s][g], 1);
                mbar_init(&full_v[s][g], 1);
                mbar_init(&empty[s][g], PAGES);          // one arrival per compute warp of the pair
            }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // query rows beyond a group's heads stay zero for the whole kernel
    for (int i = tid; i < STAGES * Q_BYTES / 16; i += THREADS) {
        const int s = i / (Q_BYTES / 16), c = i % (Q_BYTES / 16);
        *reinterpret_cast<uint4*>(stages + (size_t)s * STAGE_BYTES + 2 * PAGES * TILE_BYTES + c * 16) = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the zeros above precede the bulk copies below
    const int total = cum[n_seqs];

    auto decode = [&](int item, Item& it) {
        int lo = 0, hi = n_seqs - 1;                     // last b with cum[b] <= item
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (cum[mid] <= item) lo = mid; else hi = mid - 1;
        }
        it.b = lo;
        it.kv_len = kvl[lo];
        const int n_splits = (it.kv_len + SPLIT - 1) / SPLIT;
        int r = item - cum[lo];
        it.split = r % n_splits; r /= n_splits;
        const int pass = r % n_pass;
        it.kvh = r / n_pass;
        it.h0 = pass * NH;
        it.nh = min(NH, group - it.h0);
    };

    if (warp == CWARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int n = 0;
            for (int item = blockIdx.x; item < total; item += gridDim.x, ++n) {
                const int s = n % STAGES, g = n % GROUPS;
                // the stage held item n - 3, of the other pair: free when that pair has used it
                if (n >= STAGES && !mbar_wait(&empty[s][(n - STAGES) % GROUPS], ((n - STAGES) / (STAGES * GROUPS)) & 1, &abort_flag, status, 6)) break;
                Item it;
                decode(item, it);
                const int key_begin = it.split * SPLIT;
                const int n_pages = min(PAGES, (it.kv_len - key_begin + kPage - 1) / kPage);
                uint8_t* st = stages + (size_t)s * STAGE_BYTES;
                const uint32_t q_bytes = (uint32_t)it.nh * HD * 2;
                mbar_expect_tx(&full_k[s][g], (uint32_t)(n_pages * TILE_BYTES) + q_bytes);
                bulk_load(st + 2 * PAGES * TILE_BYTES, q + ((int64_t)it.b * n_heads + it.kvh * group + it.h0) * HD, q_bytes, &full_k[s][g]);
                for (int w = 0; w < n_pages; ++w) {
                    const int page = page_table[(int64_t)it.b * table_width + key_begin / kPage + w];
                    const int row = ((page * 2 + 0) * n_kv + it.kvh) * kPage;
                    for (int pn = 0; pn < PANELS; ++pn) tma_load_2d(&kv_map, &full_k[s][g], st + w * TILE_BYTES + pn * PANEL_BYTES, pn * 64, row);
                }
                mbar_expect_tx(&full_v[s][g], (uint32_t)(n_pages * TILE_BYTES));
                for (int w = 0; w < n_pages; ++w) {
                    const int page = page_table[(int64_t)it.b * table_width + key_begin / kPage + w];
                    const int row = ((page * 2 + 1) * n_kv + it.kvh) * kPage;
                    for (int pn = 0; pn < PANELS; ++pn) tma_load_2d(&kv_map, &full_v[s][g], st + (PAGES + w) * TILE_BYTES + pn * PANEL_BYTES, pn * 64, row);
                }
            }
        }
    } else {
        // ---------------- compute: GROUPS pairs of warps, one page per warp, items alternate between the pairs ----------------
        const float sl2 = scale * 1.4426950408889634f;
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;         // accumulator rows r0, r0 + 8; columns c0, c0 + 1
        const int grp = warp / PAGES;
        const int ctid = tid - grp * PAGES * 32;               // 0..63 within the pair
        const int wp = warp % PAGES;                           // this warp's page of an item
        bf16 (*p_s)[SPLIT] = p_all[grp];
        float (*o_s)[HD] = o_all[grp];
        float (*m_w)[NH] = m_all[grp];
        float (*l_w)[NH] = l_all[grp];
        const int bar_id = 1 + grp;                            // named barrier of this pair
        for (int n = grp; ; n += GROUPS) {
            const int item = blockIdx.x + n * gridDim.x;
            if (item >= total) break;
            const int s = n % STAGES;
            const uint32_t visit = (uint32_t)n / (STAGES * GROUPS);     // this pair's visits to this stage so far
            Item it;
            decode(item, it);
            const int key_begin = it.split * SPLIT;
            const int n_pages = min(PAGES, (it.kv_len - key_begin + kPage - 1) / kPage);
            const bool live = wp < n_pages;
            const int keys_here = live ? min(kPage, it.kv_len - key_begin - wp * kPage) : 0;
            uint8_t* st = stages + (size_t)s * STAGE_BYTES;
            const uint32_t k_base = smem_u32(st + wp * TILE_BYTES), v_base = smem_u32(st + (PAGES + wp) * TILE_BYTES);
            const bf16* q_s = reinterpret_cast<const bf16*>(st + 2 * PAGES * TILE_BYTES);

            bool ok = mbar_wait(&full_k[s][grp], visit & 1, &abort_flag, status, 6);
            // ---- scores S^T[key, head] of this warp's page ----
            float sc[4][4];
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (live && ok) {
                uint32_t qb[KS][2];
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    qb[ks][0] = *reinterpret_cast<const uint32_t*>(q_s + r0 * HD + 16 * ks + c0);
                    qb[ks][1] = *reinterpret_cast<const uint32_t*>(q_s + r0 * HD + 16 * ks + c0 + 8);
                }
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
            ok = mbar_wait(&full_v[s][grp], visit & 1, &abort_flag, status, 6) && ok;
            // Rows of the last page that hold no token yet may be anything: make them
            // zero, so that a zero weight times such a row stays zero.
            if (live && ok && keys_here < kPage) {
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
            if (lane == 0) mbar_arrive_cta(&empty[s][grp]);
            // ---- warp 1 hands its part to warp 0, which writes the item's partial result ----
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
                const int64_t row_a = ((int64_t)it.b * n_heads + it.kvh * group + it.h0 + c0) * max_splits + it.split;
                const int64_t row_b = row_a + max_splits;
#pragma unroll
                for (int mb = 0; mb < KS; ++mb) {
                    const int d = 16 * mb + r0;
                    if (c0 < it.nh) {
                        part_o[row_a * HD + d] = o[mb][0] + o_s[c0][d];
                        part_o[row_a * HD + d + 8] = o[mb][2] + o_s[c0][d + 8];
                    }
                    if (c0 + 1 < it.nh) {
                        part_o[row_b * HD + d] = o[mb][1] + o_s[c0 + 1][d];
                        part_o[row_b * HD + d + 8] = o[mb][3] + o_s[c0 + 1][d + 8];
                    }
                }
                if (lane < 4) {
                    if (c0 < it.nh) {
                        part_ml[row_a * 2] = m0;                       // in units of log2(e)
                        part_ml[row_a * 2 + 1] = l_w[0][c0] + l_w[1][c0];
                    }
                    if (c0 + 1 < it.nh) {
                        part_ml[row_b * 2] = m1;
                        part_ml[row_b * 2 + 1] = l_w[0][c0 + 1] + l_w[1][c0 + 1];
                    }
                }
            }
            if (ctid == 0) stop_s[grp] = abort_flag;                        // one decision for both warps
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");             // o_s, m_w, l_w, p_s are free again
            if (stop_s[grp]) break;
        }
    }
    __syncthreads();
    if (abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
}

// Merge of the splits of every (sequence, head), in index order.
__global__ void attn_decode_mma_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                             const int* __restrict__ kv_len_arr, bf16* __restrict__ out, int n_heads,
                                             int max_splits) {
    pdl_trigger();
    pdl_wait();
    part_o = fresh(part_o);
    part_ml = fresh(part_ml);
    const int head = blockIdx.x, b = blockIdx.y;
    const int n_splits = (kv_len_arr[b] + SPLIT - 1) / SPLIT;
    const int64_t row0 = ((int64_t)b * n_heads + head) * max_splits;
    float m = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) m = fmaxf(m, part_ml[(row0 + sp) * 2]);
    float denom = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) denom += exp2f(part_ml[(row0 + sp) * 2] - m) * part_ml[(row0 + sp) * 2 + 1];
    const float inv = n_splits > 0 ? 1.0f / denom : 0.f;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float v = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) v = fmaf(exp2f(part_ml[(row0 + sp) * 2] - m), part_o[(row0 + sp) * HD + d], v);
        out[((int64_t)b * n_heads + head) * HD + d] = __float2bfloat16_rn(v * inv);
    }
}

}  // namespace decodemma
}  // namespace wick

using namespace wick;

WICK_API int wick_attn_decode_mma_supported() { return decodemma::SUPPORTED ? 1 : 0; }
WICK_API int wick_attn_decode_mma_split() { return decodemma::SPLIT; }

// q, out: bfloat16 [n_seqs, n_heads, HD]; kv: one schedule entry's cache, bfloat16
// [kv_pages, 2, n_kv, 64, HD]; scratch: float32, n_seqs * n_heads * ceil(max_kv_len
// / 128) * (HD + 2) elements; status: device int (code 6 if a block gave up
// waiting for its copies).
WICK_API int wick_attn_decode_mma_bf16(const void* q, const void* kv, long long kv_pages, void* out, float* scratch,
                                       long long scratch_floats, const int* kv_len, int n_seqs,
                                       int max_kv_len, const int* page_table, int table_width, int n_heads, int n_kv,
                                       float scale, int* status, void* s) {
    using namespace decodemma;
    WICK_REQUIRE(SUPPORTED, "attention decode (tensor cores): head_dim %d is not 64 or 128", HD);
    WICK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads over %d kv heads", n_heads, n_kv);
    WICK_REQUIRE(n_kv <= 65535 && n_heads <= 65535, "attention: grid limit");
    WICK_REQUIRE(n_seqs <= MAX_SEQS, "attention decode (tensor cores): %d sequences, at most %d", n_seqs, MAX_SEQS);
    if (n_seqs == 0) return 0;
    const int max_splits = ceil_div(max_kv_len > 0 ? max_kv_len : 1, SPLIT);
    const long long need = (long long)n_seqs * n_heads * max_splits * (HD + 2);
    WICK_REQUIRE(scratch_floats >= need, "attention decode: scratch of %lld floats, %lld needed", scratch_floats, need);
    CUtensorMap map;
    if (int e = make_bf16_map(&map, kv, kv_pages * 2 * n_kv * kPage, HD, kPage, "attention decode")) return e;
    float* ml = scratch + (long long)n_seqs * n_heads * max_splits * HD;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised = true;
    }
    const int group = n_heads / n_kv;
    const long long items = (long long)n_seqs * n_kv * max_splits * ((group + NH - 1) / NH);   // an upper bound
    const int blocks = (int)(items < 148 ? items : 148);
    WICK_CUDA(launch(attn_decode_mma_kernel, dim3(blocks), dim3(THREADS), smem, (cudaStream_t)s, map, (const bf16*)q,
                     (bf16*)out, scratch, ml, kv_len, page_table, table_width, n_seqs, n_heads, n_kv, max_splits,
                     scale, status));
    if (int e = check_launch("attn_decode_mma")) return e;
    WICK_CUDA(launch(attn_decode_mma_merge_kernel, dim3(n_heads, n_seqs), dim3(HD), 0, (cudaStream_t)s, (const float*)scratch,
                     (const float*)ml, kv_len, (bf16*)out, n_heads, max_splits));
    return check_launch("attn_decode_mma_merge");
}
