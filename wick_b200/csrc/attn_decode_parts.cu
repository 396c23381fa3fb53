// Decode attention over the paged cache for any number of sequences (bfloat16,
// head sizes 64 and 128, up to 8 query heads per kv head): one new token per
// sequence attends to all cached positions of its sequence.
//
// How the work is cut depends on each sequence's OWN length and on nothing else, so a
// sequence's output bits do not depend on the batch it is in:
//   * the pages of a (sequence, kv head) pair are cut into PARTS of pages_per_part(n)
//     consecutive pages (two, i.e. 128 positions, up to 64 pages; more for longer
//     sequences, so that a pair never has more than 32 parts);
//   * a part is computed by ONE warp, page by page in order (scores with the keys on
//     the 16-row side of mma.sync, the probabilities turned into the second product's
//     operand inside the warp with movmatrix, running maximum, sum and accumulator in
//     registers); it leaves its result (accumulator, maximum, sum per head) in global
//     scratch;
//   * a second, small kernel (attn_decode_merge_kernel, a warp per pair and head) merges
//     a pair's parts in part order and writes the output rows.  A pair with one part is
//     written directly by the first kernel.
// Which warp computes which part is a matter of scheduling only: all parts of the step,
// in the order (sequence, kv head, part), are dealt in equal contiguous runs to the
// warps of the grid (three warps a block at head size 128, one block per SM, blocks
// first so that few parts spread over many SMs).  Every warp feeds itself: a private
// ring of four tiles (a tile is one page of keys or of values of one kv head, fetched
// by TMA into 128-byte-swizzled shared memory), filled up to four tiles ahead across
// the boundaries of its parts.  No warp waits for another one; the only waits are on
// a warp's own copies, and they are bounded.
//
// The kernel before this one (qk_norm_rope_append_kernel) has normed and rotated the
// query rows and has written the new token's key and value to the cache.  Copies of
// pages that it does not write (all but a sequence's last page) start before
// griddepcontrol.wait, i.e. while that kernel still runs.
// Formulas: wick src/model.rs:520-553.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace decodeparts {

constexpr bool SUPPORTED = WICK_HD == 64 || WICK_HD == 128;
constexpr int HD = SUPPORTED ? WICK_HD : 64;           // other head sizes: the entry point refuses, the kernel is never launched
constexpr int NH = 8;                                  // query heads of a kv head (the 8-wide side of the instruction)
constexpr int PANELS = HD / 64;
constexpr int PANEL_BYTES = kPage * 128;
constexpr int TILE_BYTES = PANELS * PANEL_BYTES;       // one page of keys (or values) of one kv head
#ifndef WICK_DECODE_WARPS
#define WICK_DECODE_WARPS 6
#endif
#ifndef WICK_DECODE_TILES
#define WICK_DECODE_TILES 2
#endif
constexpr int W = WICK_DECODE_WARPS * (128 / HD);      // warps of a block
constexpr int T = WICK_DECODE_TILES;                   // tiles of a warp's ring
constexpr int THREADS = W * 32;
constexpr int KS = HD / 16;
constexpr int EPL = HD / 32;                           // elements of a head row per lane
constexpr int PART_PAGES = 2;                          // pages of a part (sequences of up to PART_PAGES * MAX_PARTS pages)
constexpr int MAX_PARTS = 8;
constexpr int MAX_SEQS = 1024;
constexpr int MAX_SPLITS = 8;                          // partial sums of the projection that the kernel adds up
constexpr int REC = HD + 2;                            // a head's record in the scratch: accumulator, maximum, sum
constexpr int ROWS_BYTES = (NH + 2) * HD * 2;          // a warp's query rows and the new token's key and value, bfloat16
constexpr int SMEM_BYTES = W * T * TILE_BYTES + W * ROWS_BYTES + 1024;
typedef __nv_bfloat16 bf16;

// Pages of one part of a sequence of n_pages pages: a function of the sequence's own length.
__host__ __device__ inline int pages_per_part(int n_pages) {
    const int cap = PART_PAGES * MAX_PARTS;
    return n_pages <= cap ? PART_PAGES : PART_PAGES * ((n_pages + cap - 1) / cap);
}
__host__ __device__ inline int parts_of(int n_pages) {
    const int pp = pages_per_part(n_pages);
    return (n_pages + pp - 1) / pp;
}

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
// An 8 x 8 matrix of 16-bit elements, held by the warp one row per four lanes (a lane has
// two neighbouring elements of its row): the transposed matrix in the same layout.
__device__ __forceinline__ uint32_t transpose8x8(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// Byte offset, inside a page tile, of the 16-byte chunk `chunk` (8 elements) of row `row`.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * PANEL_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
__device__ __forceinline__ float ld_cg(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 2^(a - b) for maxima that may be -inf (nothing seen yet): then the weight is 0.
__device__ __forceinline__ float weight(float a, float b) { return a == -INFINITY ? 0.f : exp2f(a - b); }

// One head of a pair: its P parts' records folded in part order into a running maximum M, sum
// l and accumulator o (a lane holds HD / 32 dims):
//   M' = max(M, m_p);  l = l 2^(M - M') + l_p 2^(m_p - M');  o likewise;  out = o / l.
// word(p, i) gives word i of part p's record (i < HD: the accumulator, HD: the maximum, HD + 1:
// the sum).  Every product and sum is rounded on its own, so that the result does not depend on
// which kernel this is compiled into.
template <typename Word>
__device__ __forceinline__ void merge_head(Word word, int P, int lane, bf16* dst) {
    float bo[MAX_PARTS][EPL], bm[MAX_PARTS], bl[MAX_PARTS];
#pragma unroll
    for (int p = 0; p < MAX_PARTS; ++p) {
        const int pp = min(p, P - 1);
        bm[p] = word(pp, HD);
        bl[p] = word(pp, HD + 1);
#pragma unroll
        for (int e = 0; e < EPL; ++e) bo[p][e] = word(pp, lane + 32 * e);
    }
    float M = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = 0.f;
#pragma unroll
    for (int p = 0; p < MAX_PARTS; ++p) {
        if (p < P) {
            const float mn = fmaxf(M, bm[p]);
            const float a = weight(M, mn), w = weight(bm[p], mn);
            l = __fadd_rn(__fmul_rn(l, a), __fmul_rn(bl[p], w));
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[e] = __fadd_rn(__fmul_rn(o[e], a), __fmul_rn(bo[p][e], w));
            M = mn;
        }
    }
    const float inv = l > 0.f ? __fdiv_rn(1.0f, l) : 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[lane + 32 * e] = __float2bfloat16_rn(__fmul_rn(o[e], inv));
}

// A warp's place in its run of parts: the part it is at and the page inside it.
struct Walk {
    int u;                     // the part's number among all parts of the step
    int b, kvh, part;          // its sequence, kv head and number within the pair
    int len, n_pages, parts;   // of sequence b
    int page, page_end;        // the page (of the sequence) it is at, and the part's end
    int is_v;                  // the tile of that page: keys (0) or values (1)
};

// cum, lens: the block's copies (shared memory) of the parts before each sequence and of the lengths.
__device__ __forceinline__ void open_part(Walk& w, const int* cum, const int* lens, int n_kv) {
    while (w.u >= cum[w.b + 1]) ++w.b;                 // (parts are visited in order: b only moves forward)
    w.len = lens[w.b];
    w.n_pages = (w.len + kPage - 1) / kPage;
    const int pp = pages_per_part(w.n_pages);
    w.parts = (w.n_pages + pp - 1) / pp;
    const int local = w.u - cum[w.b];
    w.kvh = local / w.parts;
    w.part = local % w.parts;
    w.page = w.part * pp;
    w.page_end = min(w.n_pages, w.page + pp);
    w.is_v = 0;
}

// What the kernel is given for the new token: either its query rows, normed and rotated (and
// its key and value are in the cache already), or the projection's float32 partial sums, from
// which a warp makes a pair's query rows when it comes to that pair, and the warp that has the
// pair's last part the new key and value as well (wick src/model.rs:475-480): it writes them
// to the cache and patches them into the tiles it has fetched (the copy may have read those
// rows before or after they were written).
struct Projection {
    const float* sums;         // [splits, n_seqs, (n_heads + 2 n_kv) HD], or null
    int splits;
    int64_t split_stride;
    const float* q_w;          // per-head norm weights [HD], or null
    const float* k_w;
    float eps;
    const float* cos_t;        // [n_seqs, HD / 2], or null
    const float* sin_t;
    bf16* kv;                  // the cache, for the new token's rows
    int write_kv;
};

// PAIR: the form for few pairs (up to some 400; fewer for long sequences: the host decides by
// measured rules).  A block takes one pair and its warps the pair's parts; the block makes the new
// token's rows once, all warps at it (a row or two each, one trip to the L2 cache), and when
// all parts are done its warps merge the pair's records, a head each: one launch.  Otherwise
// (persistent form) all parts of the step are dealt to the warps of one block per SM, and the
// merge kernel follows.  Which form runs changes no bit: a part is computed by one warp in the
// same way, and the parts are folded in the same order with the same operations.
template <bool PREP, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
attn_decode_parts_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* q, Projection proj, bf16* __restrict__ out,
                         const int* __restrict__ kv_len_arr, const int* __restrict__ page_table, int table_width,
                         int n_seqs, int n_heads, int n_kv, float scale, float* partials, int part_stride, int kv_pages,
                         int* status) {
    constexpr int NW = W;                              // warps of a block
    constexpr int TT = T;                              // tiles of a warp's ring
    constexpr int u_step = PAIR ? W : 1;               // from a warp's part to its next one
    extern __shared__ uint8_t smem_raw[];
    __shared__ int cum[(PAIR ? 1 : MAX_SEQS) + 1];     // parts of the sequences before each sequence (times kv heads)
    __shared__ int lens[PAIR ? 1 : MAX_SEQS];          // the sequences' lengths (0: left out)
    __shared__ uint64_t full[NW][TT];
    __shared__ int abort_flag;

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = n_heads / n_kv;
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    if (tid == 0) {
        abort_flag = 0;
        for (int w = 0; w < NW; ++w)
            for (int t = 0; t < TT; ++t) mbar_init(&full[w][t], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // b_base: the sequence that index 0 of cum / lens stands for (PAIR: the pair's own, the only one the block knows)
    int b_base = 0, u0 = 0, u1 = 0, my_parts = 0;
    if (PAIR) {
        const int pair = (int)blockIdx.x;
        b_base = pair / n_kv;
        const int len = kv_len_arr[b_base];            // (in place before the step's first kernel starts, see below)
        const int n_pages = (len + kPage - 1) / kPage;
        const bool fits = len > 0 && n_pages <= table_width && parts_of(n_pages) <= part_stride;
        if (len > 0 && !fits && tid == 0) atomicCAS(status, 0, 10);
        my_parts = fits ? parts_of(n_pages) : 0;
        if (tid == 0) {
            lens[0] = fits ? len : 0;
            cum[0] = 0;
            cum[1] = my_parts * n_kv;
        }
        u0 = (pair % n_kv) * my_parts + warp;          // this warp's parts: warp, warp + W, ...
        u1 = (pair % n_kv) * my_parts + my_parts;
    } else if (warp == 0) {
        // The step's lengths are in place before the step's first kernel starts (the host or
        // the kernel that prepares a step writes them; neither is the kernel before this one).
        int before = 0;
        for (int s0 = 0; s0 < n_seqs; s0 += 32) {
            const int s = s0 + lane;
            int mine = 0;
            if (s < n_seqs) {
                const int len = kv_len_arr[s];
                const int n_pages = (len + kPage - 1) / kPage;
                if (len > 0 && n_pages <= table_width && parts_of(n_pages) <= part_stride) mine = parts_of(n_pages) * n_kv;
                else if (len > 0) atomicCAS(status, 0, 10);      // longer than its page table or than the scratch allows: left out, and said so
                lens[s] = mine ? len : 0;
            }
            int upto = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, upto, o);
                if (lane >= o) upto += t;
            }
            if (s < n_seqs) cum[s + 1] = before + upto;
            before += __shfl_sync(0xffffffffu, upto, 31);
        }
        if (lane == 0) cum[0] = 0;
    }
    __syncthreads();

    if (!PAIR) {
        // This warp's run of parts.
        const int U = cum[n_seqs];
        const int64_t S = (int64_t)gridDim.x * W, slot = (int64_t)warp * gridDim.x + blockIdx.x;
        u0 = (int)(slot * U / S);
        u1 = (int)((slot + 1) * U / S);
        if (u0 >= u1) return;
    }
    const bool work = u0 < u1;                         // (PAIR: a warp without a part still helps with the rows and the merge)

    uint8_t* ring = tiles + (size_t)warp * TT * TILE_BYTES;
    Walk pw, cw;                                       // where the copies are, where the computation is
    {
        int lo = 0, hi = (PAIR ? 1 : n_seqs) - 1;      // the sequence of part u0: the last b with cum[b] <= u0
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (cum[mid] <= u0) lo = mid;
            else hi = mid - 1;
        }
        pw.u = u0;
        pw.b = lo;
        if (work) open_part(pw, cum, lens, n_kv);
        cw = pw;
    }
    // The page ids of a part: lane j holds the part's j-th page (a part of more than 32 pages
    // asks for the others one by one).  The ids of the part after the one being copied are
    // asked for when that one is opened, so that they have arrived when they are needed: a
    // load from the page table costs a trip to the L2 cache, and nothing else runs in this
    // warp meanwhile.
    auto page_ids = [&](const Walk& w) -> int {
        const int j = w.page + lane;
        return j < w.page_end ? page_table[(int64_t)(b_base + w.b) * table_width + j] : 0;
    };
    Walk nw = pw;                                      // the part after pw's
    int ids = work ? page_ids(pw) : 0, ids_next = 0, ids_first = pw.page;
    auto peek_next = [&]() {
        nw.u = pw.u + u_step;
        nw.b = pw.b;
        if (nw.u < u1) {
            open_part(nw, cum, lens, n_kv);
            ids_next = page_ids(nw);
        }
    };
    if (work) peek_next();
    uint32_t issued = 0, consumed = 0;
    bool dead = false;

    // Start the copy of the next tile, if there is one, the ring has room, and (before the
    // wait for the kernel that writes the new token's key and value) it is not a sequence's
    // last page.
    auto issue = [&](bool after_wait) -> bool {
        if (dead || pw.u >= u1 || issued - consumed >= (uint32_t)TT) return false;
        if (!PREP && !after_wait && pw.page == pw.n_pages - 1) return false;   // (that kernel writes this page)
        const int j = pw.page - ids_first;
        const int page = j < 32 ? __shfl_sync(0xffffffffu, ids, j) : page_table[(int64_t)(b_base + pw.b) * table_width + pw.page];
        if (page < 0 || page >= kv_pages) {            // a page outside the cache: give up, say so
            if (lane == 0) {
                *(volatile int*)&abort_flag = 1;
                atomicCAS(status, 0, 10);
            }
            dead = true;
            return false;
        }
        const uint32_t s = issued % TT;
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tile's last readers (this warp) are done
            uint8_t* dst = ring + s * TILE_BYTES;
            mbar_expect_tx(&full[warp][s], (uint32_t)TILE_BYTES);
            for (int pn = 0; pn < PANELS; ++pn)
                tma_load_2d(&kv_map, &full[warp][s], dst + pn * PANEL_BYTES, pn * 64, ((page * 2 + pw.is_v) * n_kv + pw.kvh) * kPage);
        }
        ++issued;
        if (!pw.is_v) pw.is_v = 1;
        else {
            pw.is_v = 0;
            if (++pw.page == pw.page_end) {
                pw = nw;                               // (pw.u becomes u1 after the run's last part)
                ids = ids_next;
                ids_first = pw.page;
                if (pw.u < u1) peek_next();
            }
        }
        return true;
    };
    while (issue(false)) {}
    pdl_wait();                                        // the query rows (or the projection's sums they are made from)
    q = fresh(q);

    const float sl2 = scale * 1.4426950408889634f;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;     // accumulator rows r0, r0 + 8; columns c0, c0 + 1
    int q_of = -1;                                     // the pair whose query rows are in qb
    uint32_t qb[KS][2];
    bf16 (*rows_s)[HD] = reinterpret_cast<bf16 (*)[HD]>(tiles + (size_t)NW * TT * TILE_BYTES + (size_t)(PAIR ? 0 : warp) * ROWS_BYTES);
    // rows_s[0 .. NH - 1]: the pair's query rows; rows_s[NH], rows_s[NH + 1]: the new key and value
    // (a set of rows per warp; PAIR: one set for the block)

    // One head row from the projection's partial sums: summed in index order, normed (if w),
    // rotated (if rot), as bfloat16 into dst.  A lane holds elements lane, lane + 32, ...: both
    // members of every rotated pair (i, i + HD / 2).  TWO rows at a time, so that a round trip
    // to the L2 cache serves both.
    auto make_rows = [&](int b, int64_t off_a, int64_t off_b, bool has_b, const float* w_a, const float* w_b, bool rot_a,
                         bool rot_b, bf16* dst_a, bf16* dst_b) {
        constexpr int half = HD / 2;
        const float* row = proj.sums + (int64_t)b * (n_heads + 2 * n_kv) * HD;
        float raw[2][MAX_SPLITS][EPL];
#pragma unroll
        for (int sp = 0; sp < MAX_SPLITS; ++sp)
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                raw[0][sp][e] = sp < proj.splits ? ld_cg(row + sp * proj.split_stride + off_a + lane + 32 * e) : 0.f;
                raw[1][sp][e] = (has_b && sp < proj.splits) ? ld_cg(row + sp * proj.split_stride + off_b + lane + 32 * e) : 0.f;
            }
        float cs[EPL / 2], sn[EPL / 2];
#pragma unroll
        for (int e = 0; e < EPL / 2; ++e) {
            const bool rot = proj.cos_t && (rot_a || rot_b);
            cs[e] = rot ? ld_cg(proj.cos_t + (int64_t)b * half + lane + 32 * e) : 1.f;
            sn[e] = rot ? ld_cg(proj.sin_t + (int64_t)b * half + lane + 32 * e) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (r == 1 && !has_b) break;
            const float* w = r ? w_b : w_a;
            const bool rot = proj.cos_t && (r ? rot_b : rot_a);
            bf16* dst = r ? dst_b : dst_a;
            float v[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                float x = raw[r][0][e];
#pragma unroll
                for (int sp = 1; sp < MAX_SPLITS; ++sp)
                    if (sp < proj.splits) x = __fadd_rn(x, raw[r][sp][e]);
                v[e] = x;
            }
            float sc = 1.f;
            if (w) {
                float ss = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) ss = __fmaf_rn(v[e], v[e], ss);
                ss = warp_sum(ss);
                sc = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)HD), proj.eps)));
            }
#pragma unroll
            for (int e = 0; e < EPL / 2; ++e) {
                const int i = lane + 32 * e;             // < HD / 2; its partner is i + HD / 2
                float x = v[e], y = v[e + EPL / 2];
                if (w) {
                    x = __fmul_rn(__fmul_rn(x, sc), w[i]);
                    y = __fmul_rn(__fmul_rn(y, sc), w[i + half]);
                }
                if (rot) {
                    const float rx = __fsub_rn(__fmul_rn(x, cs[e]), __fmul_rn(y, sn[e])), ry = __fadd_rn(__fmul_rn(y, cs[e]), __fmul_rn(x, sn[e]));
                    x = rx;
                    y = ry;
                }
                dst[i] = __float2bfloat16_rn(x);
                dst[i + half] = __float2bfloat16_rn(y);
            }
        }
    };

    if (PAIR) {
        if (PREP && my_parts > 0) {
            // the pair's rows, a warp at one or two of them: query heads 0 .. group - 1, then the new key and value
            const int kvh = (int)blockIdx.x % n_kv, n_rows = group + (proj.write_kv ? 2 : 0);
            auto offset = [&](int ri) { return ri < group ? (int64_t)(kvh * group + ri) * HD : (int64_t)(n_heads + (ri - group) * n_kv + kvh) * HD; };
            auto norm_w = [&](int ri) { return ri < group ? proj.q_w : (ri == group ? proj.k_w : (const float*)nullptr); };
            auto dest = [&](int ri) { return ri < group ? rows_s[ri] : rows_s[NH + ri - group]; };
            const int ra = warp, rb = warp + W;
            if (ra < n_rows)
                make_rows(b_base, offset(ra), offset(min(rb, n_rows - 1)), rb < n_rows, norm_w(ra), norm_w(min(rb, n_rows - 1)),
                          ra <= group, rb <= group, dest(ra), dest(min(rb, n_rows - 1)));
        }
        __syncthreads();
    }

    while (cw.u < u1 && !dead) {
        const int b = b_base + cw.b, kvh = cw.kvh, pair = b * n_kv + kvh;
        const bool owner = PREP && proj.write_kv && cw.part == cw.parts - 1;   // this part ends with the new token
        if (pair != q_of) {
            if (PREP) {
                if (!PAIR) {
                    for (int h = 0; h < group; h += 2)
                        make_rows(b, (int64_t)(kvh * group + h) * HD, (int64_t)(kvh * group + h + 1) * HD, h + 1 < group, proj.q_w,
                                  proj.q_w, true, true, rows_s[h], rows_s[h + 1]);
                    __syncwarp();
                }
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    qb[ks][0] = r0 < group ? *reinterpret_cast<const uint32_t*>(&rows_s[r0][16 * ks + c0]) : 0u;
                    qb[ks][1] = r0 < group ? *reinterpret_cast<const uint32_t*>(&rows_s[r0][16 * ks + c0 + 8]) : 0u;
                }
            } else {
                // Q^T as the 8-wide operand: head r0 of the group, dims 16 ks + c0 (+ 1, + 8, + 9)
                const bf16* row = q + ((int64_t)b * n_heads + kvh * group + r0) * HD;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    qb[ks][0] = r0 < group ? ld_cg_u32(row + 16 * ks + c0) : 0u;
                    qb[ks][1] = r0 < group ? ld_cg_u32(row + 16 * ks + c0 + 8) : 0u;
                }
            }
            q_of = pair;
        }
        if (owner) {
            // the new token's key (normed, rotated) and value: into the cache, for the steps to come
            if (!PAIR) {
                make_rows(b, (int64_t)(n_heads + kvh) * HD, (int64_t)(n_heads + n_kv + kvh) * HD, true, proj.k_w, nullptr, true, false,
                          rows_s[NH], rows_s[NH + 1]);
                __syncwarp();
            }
            const int pos = cw.len - 1;
            const int page = page_table[(int64_t)b * table_width + pos / kPage];
            if (page >= 0 && page < kv_pages && lane < 2 * (HD / 8)) {
                const int is_v = lane / (HD / 8), chunk = lane % (HD / 8);
                bf16* dst = proj.kv + ((((int64_t)page * 2 + is_v) * n_kv + kvh) * kPage + (pos % kPage)) * HD;
                reinterpret_cast<uint4*>(dst)[chunk] = reinterpret_cast<const uint4*>(rows_s[NH + is_v])[chunk];
            }
        }
        // the part's running result: maxima in units of log2 e, for heads c0 and c0 + 1
        float mr0 = -INFINITY, mr1 = -INFINITY, lr0 = 0.f, lr1 = 0.f;
        float acc[KS][4];                              // O^T[dim, head]: dims 16 mb + r0 (+ 8), heads c0, c0 + 1
#pragma unroll
        for (int mb = 0; mb < KS; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;

        for (int page = cw.page; page < cw.page_end; ++page) {
            const int keys_here = min(kPage, cw.len - page * kPage);
            while (issue(true)) {}
            // ---- scores S^T[key, head] of the page ----
            uint32_t s = consumed % TT;
            bool ok = mbar_wait(&full[warp][s], (consumed / TT) & 1, &abort_flag, status, 8);
            const uint32_t k_base = smem_u32(ring + s * TILE_BYTES);
            const int new_row = (owner && page == cw.n_pages - 1) ? (cw.len - 1) % kPage : -1;
            if (new_row >= 0 && ok) {
                if (lane < HD / 8)
                    *reinterpret_cast<uint4*>(ring + s * TILE_BYTES + tile_off(new_row, lane)) = reinterpret_cast<const uint4*>(rows_s[NH])[lane];
                __syncwarp();
            }
            float sc[4][4];
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (ok) {
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
                    sc[mb][0] = ka < keys_here ? __fmul_rn(sc[mb][0], sl2) : -INFINITY;
                    sc[mb][1] = ka < keys_here ? __fmul_rn(sc[mb][1], sl2) : -INFINITY;
                    sc[mb][2] = kb < keys_here ? __fmul_rn(sc[mb][2], sl2) : -INFINITY;
                    sc[mb][3] = kb < keys_here ? __fmul_rn(sc[mb][3], sl2) : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(sc[mb][0], sc[mb][2]));
                    mx1 = fmaxf(mx1, fmaxf(sc[mb][1], sc[mb][3]));
                }
            }
            __syncwarp();
            ++consumed;                                // the keys are read: their tile may be filled again
            while (issue(true)) {}
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            }
            // a page always holds at least one position, so the new maxima are finite
            const float n0 = fmaxf(mr0, mx0), n1 = fmaxf(mr1, mx1);
            const float a0 = weight(mr0, n0), a1 = weight(mr1, n1);
            float l0 = 0.f, l1 = 0.f;
            uint32_t pb[4][2];                         // P[key, head] as the 8-wide operand of the second product
            if (ok) {
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) {
                    const float p0 = exp2f(__fsub_rn(sc[mb][0], n0)), p1 = exp2f(__fsub_rn(sc[mb][1], n1));
                    const float p2 = exp2f(__fsub_rn(sc[mb][2], n0)), p3 = exp2f(__fsub_rn(sc[mb][3], n1));
                    l0 = __fadd_rn(l0, __fadd_rn(p0, p2));
                    l1 = __fadd_rn(l1, __fadd_rn(p1, p3));
                    // rows = keys (r0, r0 + 8), columns = heads (c0, c0 + 1) -> rows = heads, columns = keys
                    pb[mb][0] = transpose8x8(pack_bf16(p0, p1));
                    pb[mb][1] = transpose8x8(pack_bf16(p2, p3));
                }
            }
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, o);
                l1 += __shfl_xor_sync(0xffffffffu, l1, o);
            }
            lr0 = __fmaf_rn(lr0, a0, l0);
            lr1 = __fmaf_rn(lr1, a1, l1);
            mr0 = n0;
            mr1 = n1;
#pragma unroll
            for (int mb = 0; mb < KS; ++mb) {
                acc[mb][0] *= a0;
                acc[mb][2] *= a0;
                acc[mb][1] *= a1;
                acc[mb][3] *= a1;
            }
            // ---- O^T[dim, head] += V^T[dim, key] P[key, head] ----
            s = consumed % TT;
            ok = mbar_wait(&full[warp][s], (consumed / TT) & 1, &abort_flag, status, 8) && ok;
            uint8_t* v_tile = ring + s * TILE_BYTES;
            if (ok && new_row >= 0 && lane < HD / 8)
                *reinterpret_cast<uint4*>(v_tile + tile_off(new_row, lane)) = reinterpret_cast<const uint4*>(rows_s[NH + 1])[lane];
            if (ok && new_row >= 0) __syncwarp();
            if (ok && keys_here < kPage) {
                // Rows of the last page that hold no token yet may be anything: make them zero,
                // so that a zero weight times such a row stays zero.
                for (int i = lane; i < (kPage - keys_here) * (HD / 8); i += 32) {
                    const int row = keys_here + i / (HD / 8), chunk = i % (HD / 8);
                    *reinterpret_cast<uint4*>(v_tile + tile_off(row, chunk)) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            if (ok) {
                const uint32_t v_base = smem_u32(v_tile);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int key = 16 * j + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
                    for (int mb = 0; mb < KS; ++mb) {
                        uint32_t a[4];
                        ldsm_x4_trans(a, v_base + tile_off(key, 2 * mb + ((lane >> 3) & 1)));
                        mma16816(acc[mb], a, pb[j][0], pb[j][1]);
                    }
                }
            }
            __syncwarp();
            ++consumed;                                // the values are read
            if (!ok) dead = true;
        }
        if (dead) break;

        if (cw.parts == 1) {
            // the pair's only part: straight to the output rows
            const float i0 = lr0 > 0.f ? __fdiv_rn(1.0f, lr0) : 0.f, i1 = lr1 > 0.f ? __fdiv_rn(1.0f, lr1) : 0.f;
            bf16* o0 = out + ((int64_t)b * n_heads + kvh * group + c0) * HD;
#pragma unroll
            for (int mb = 0; mb < KS; ++mb) {
                const int d = 16 * mb + r0;
                if (c0 < group) {
                    o0[d] = __float2bfloat16_rn(__fmul_rn(acc[mb][0], i0));
                    o0[d + 8] = __float2bfloat16_rn(__fmul_rn(acc[mb][2], i0));
                }
                if (c0 + 1 < group) {
                    o0[HD + d] = __float2bfloat16_rn(__fmul_rn(acc[mb][1], i1));
                    o0[HD + d + 8] = __float2bfloat16_rn(__fmul_rn(acc[mb][3], i1));
                }
            }
        } else {
            // the part's record, for the merge
            float* rec = partials + ((int64_t)pair * part_stride + cw.part) * group * REC;
#pragma unroll
            for (int mb = 0; mb < KS; ++mb) {
                const int d = 16 * mb + r0;
                if (c0 < group) {
                    rec[c0 * REC + d] = acc[mb][0];
                    rec[c0 * REC + d + 8] = acc[mb][2];
                }
                if (c0 + 1 < group) {
                    rec[(c0 + 1) * REC + d] = acc[mb][1];
                    rec[(c0 + 1) * REC + d + 8] = acc[mb][3];
                }
            }
            if (r0 == 0) {
                if (c0 < group) { rec[c0 * REC + HD] = mr0; rec[c0 * REC + HD + 1] = lr0; }
                if (c0 + 1 < group) { rec[(c0 + 1) * REC + HD] = mr1; rec[(c0 + 1) * REC + HD + 1] = lr1; }
            }
        }
        cw.u += u_step;
        if (cw.u < u1) open_part(cw, cum, lens, n_kv);
    }
    if (PAIR) {
        __syncthreads();                               // every part's record is written (and visible to this block)
        if (my_parts > 1 && !abort_flag) {
            const int pair = (int)blockIdx.x;
            for (int h = warp; h < group; h += W) {
                const float* first = partials + ((int64_t)pair * part_stride * group + h) * REC;
                merge_head([&](int p, int i) { return ld_cg(first + (int64_t)p * group * REC + i); }, my_parts, lane,
                           out + ((int64_t)(pair / n_kv) * n_heads + (pair % n_kv) * group + h) * HD);
            }
        }
    }
    if (abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000); // copies in flight land before the warp leaves
    }
}

// The records of a pair's parts, merged in part order: a warp per (pair, head), a lane per
// HD / 32 dims.  With running maximum M, sum l and accumulator o, part p is folded in as
//   M' = max(M, m_p);  l = l 2^(M - M') + l_p 2^(m_p - M');  o likewise;
// and out = o / l.  All of a pair's records are asked for at once (one trip to the L2 cache).
// Pairs with one part were written by the first kernel and are skipped.
__global__ void __launch_bounds__(128)
attn_decode_merge_kernel(const float* partials, bf16* __restrict__ out, const int* __restrict__ kv_len_arr, int table_width,
                         int n_seqs, int n_heads, int n_kv, int part_stride) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int group = n_heads / n_kv;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);       // (pair, head)
    if (item >= n_seqs * n_heads) return;
    const int pair = item / group, h = item % group;
    const int len = kv_len_arr[pair / n_kv];           // (the step's lengths are in place before the step starts)
    const int n_pages = (len + kPage - 1) / kPage;
    if (len <= 0 || n_pages > table_width) return;
    const int P = parts_of(n_pages);
    if (P < 2 || P > part_stride) return;
    pdl_wait();                                        // the records
    partials = fresh(partials);
    const float* first = partials + ((int64_t)pair * part_stride * group + h) * REC;
    merge_head([&](int p, int i) { return ld_cg(first + (int64_t)p * group * REC + i); }, P, lane,
               out + ((int64_t)(pair / n_kv) * n_heads + (pair % n_kv) * group + h) * HD);
}

}  // namespace decodeparts
}  // namespace wick

using namespace wick;

// Whether the kernel takes this problem: head size 64 or 128, at most 8 query heads per kv head.
WICK_API int wick_attn_decode_parts_supported(int n_seqs, int n_heads, int n_kv) {
    using namespace decodeparts;
    if (!SUPPORTED || n_kv <= 0 || n_heads % n_kv != 0 || n_heads / n_kv > NH) return 0;
    return n_seqs <= MAX_SEQS ? 1 : 0;
}

// Scratch for a step of n_seqs sequences of at most max_kv_len positions: float32 words for
// every part's record.
static int part_stride_for(int max_kv_len) {
    using namespace decodeparts;
    const int pages = ceil_div(max_kv_len > 0 ? max_kv_len : 1, kPage);
    if (pages <= PART_PAGES) return 1;
    const int halves = ceil_div(pages, PART_PAGES);
    return halves < MAX_PARTS ? halves : MAX_PARTS;
}

WICK_API long long wick_attn_decode_parts_scratch(int n_seqs, int n_heads, int n_kv, int max_kv_len) {
    using namespace decodeparts;
    return (long long)n_seqs * n_kv * part_stride_for(max_kv_len) * (n_heads / n_kv) * REC;
}

static int launch_parts(bool prep, const void* q, decodeparts::Projection proj, const void* kv, long long kv_pages, void* out,
                        float* scratch, long long scratch_words, const int* kv_len, int n_seqs, int max_kv_len,
                        const int* page_table, int table_width, int n_heads, int n_kv, float scale, int* status, void* s) {
    using namespace decodeparts;
    WICK_REQUIRE(SUPPORTED, "attention decode: head_dim %d is not 64 or 128", (int)WICK_HD);
    WICK_REQUIRE(wick_attn_decode_parts_supported(n_seqs, n_heads, n_kv), "attention decode: %d sequences, %d heads over %d kv heads is beyond this kernel", n_seqs, n_heads, n_kv);
    WICK_REQUIRE(kv_pages > 0 && kv_pages * 2 * n_kv * kPage < (1ll << 31), "attention decode: a cache of %lld pages is beyond the kernel's 31-bit row index", kv_pages);
    if (n_seqs == 0) return 0;
    const long long need = wick_attn_decode_parts_scratch(n_seqs, n_heads, n_kv, max_kv_len);
    WICK_REQUIRE(scratch_words >= need, "attention decode: scratch of %lld words given, %lld needed", scratch_words, need);
    CUtensorMap map;
    if (int e = make_bf16_map(&map, kv, kv_pages * 2 * n_kv * kPage, HD, kPage, "attention decode")) return e;
    const int stride = part_stride_for(max_kv_len);
    const long long most = (long long)n_seqs * n_kv * stride;
    const int sms = sm_count();
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_parts_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_parts_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_parts_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        WICK_CUDA(cudaFuncSetAttribute(attn_decode_parts_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        raised = true;
    }
    const long long pairs = (long long)n_seqs * n_kv;
    const int pages = ceil_div(max_kv_len > 0 ? max_kv_len : 1, kPage);
    static int force = -2;                             // WICK_B200_PAIR_DECODE=0/1: never / whenever possible (for measurements)
    if (force == -2) force = getenv("WICK_B200_PAIR_DECODE") ? atoi(getenv("WICK_B200_PAIR_DECODE")) : -1;
    // Measured (8 kv heads of 128, one B200): a block per pair costs about 5 us + 0.4 us a page whatever the
    // number of pairs, until the SMs that have a pair cannot keep the memory busy between them; the persistent
    // form costs about 9 us + the step's bytes at 5 TB/s.
    const bool pays = pages <= 16 || pairs >= 96 || (pairs >= 24 && pages <= 24) || (pairs >= 48 && pages <= 32);
    // More pairs than SMs, up to some 400: the blocks run in waves; that still beats the persistent form, whose
    // warps then have one or two parts each, unless the last wave is mostly empty.
    const long long waves = (pairs + sms - 1) / sms;
    const bool waves_pay = pairs <= 400 && pairs * 10 >= waves * sms * 6;
    const bool pair_form = force >= 0 ? force == 1 : (pairs <= sms ? pays : waves_pay);
    if (pair_form) {
        // Few pairs of short parts: a block per pair, its warps at the pair's parts, merged by the block itself.
        // (Longer parts, or more pairs than SMs, want the self-fed warps of the persistent form.)
        if (prep)
            WICK_CUDA(launch(attn_decode_parts_kernel<true, true>, dim3((unsigned)pairs), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)s, map,
                             (const bf16*)q, proj, (bf16*)out, kv_len, page_table, table_width, n_seqs, n_heads, n_kv, scale, scratch,
                             stride, (int)kv_pages, status));
        else
            WICK_CUDA(launch(attn_decode_parts_kernel<false, true>, dim3((unsigned)pairs), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)s, map,
                             (const bf16*)q, proj, (bf16*)out, kv_len, page_table, table_width, n_seqs, n_heads, n_kv, scale, scratch,
                             stride, (int)kv_pages, status));
        return check_launch("attn_decode_parts (a block per pair)");
    }
    // As many blocks as there can be parts, up to one per SM (who computes a part changes no bit).
    const int grid = (int)(most < sms ? most : sms);
    if (prep)
        WICK_CUDA(launch(attn_decode_parts_kernel<true, false>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)s, map,
                         (const bf16*)q, proj, (bf16*)out, kv_len, page_table, table_width, n_seqs, n_heads, n_kv, scale, scratch,
                         stride, (int)kv_pages, status));
    else
        WICK_CUDA(launch(attn_decode_parts_kernel<false, false>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)s, map,
                         (const bf16*)q, proj, (bf16*)out, kv_len, page_table, table_width, n_seqs, n_heads, n_kv, scale, scratch,
                         stride, (int)kv_pages, status));
    if (int e = check_launch("attn_decode_parts")) return e;
    if (stride > 1) {
        WICK_CUDA(launch(attn_decode_merge_kernel, dim3(ceil_div((long long)n_seqs * n_heads, 4)), dim3(128), 0, (cudaStream_t)s,
                         (const float*)scratch, (bf16*)out, kv_len, table_width, n_seqs, n_heads, n_kv, stride));
        return check_launch("attn_decode_merge");
    }
    return 0;
}

// q, out: bfloat16 [n_seqs, n_heads, HD]; kv: one schedule entry's cache, bfloat16
// [kv_pages, 2, n_kv, 64, HD], the new token's key and value already in it; kv_len: positions
// per sequence including the new token; scratch: float32 (see above); status: device int (code
// 8 if a warp gave up waiting for its copies, 10 if a length or a page lies outside what it was
// given).  Two launches: the parts, then (if any sequence can have more than one part) the merge.
WICK_API int wick_attn_decode_parts_bf16(const void* q, const void* kv, long long kv_pages, void* out, float* scratch,
                                         long long scratch_words, const int* kv_len, int n_seqs, int max_kv_len,
                                         const int* page_table, int table_width, int n_heads, int n_kv, float scale,
                                         int* status, void* s) {
    decodeparts::Projection none = {};
    return launch_parts(false, q, none, kv, kv_pages, out, scratch, scratch_words, kv_len, n_seqs, max_kv_len, page_table,
                        table_width, n_heads, n_kv, scale, status, s);
}

// The same from the q/k/v projection's float32 partial sums [splits, n_seqs, (n_heads + 2 n_kv) HD]:
// the kernel adds them up, norms q and k per head (q_w, k_w: [HD] or null), rotates them (cos_t,
// sin_t: [n_seqs, HD / 2] or null), writes the new key and value to the cache (unless write_kv is
// 0: the cache then holds them already) and attends.
WICK_API int wick_attn_decode_parts_fused_bf16(const float* sums, int splits, const float* q_w, const float* k_w, float eps,
                                               const float* cos_t, const float* sin_t, int write_kv, void* kv,
                                               long long kv_pages, void* out, float* scratch, long long scratch_words,
                                               const int* kv_len, int n_seqs, int max_kv_len, const int* page_table,
                                               int table_width, int n_heads, int n_kv, float scale, int* status, void* s) {
    using namespace decodeparts;
    WICK_REQUIRE(splits >= 1 && splits <= MAX_SPLITS, "attention decode: %d partial sums, at most %d", splits, MAX_SPLITS);
    WICK_REQUIRE((q_w == nullptr) == (k_w == nullptr) && (cos_t == nullptr) == (sin_t == nullptr), "attention decode: q and k norm weights come together, and so do the rotation tables");
    Projection proj = {sums, splits, (int64_t)n_seqs * (n_heads + 2 * n_kv) * HD, q_w, k_w, eps, cos_t, sin_t, (bf16*)kv, write_kv};
    return launch_parts(true, nullptr, proj, kv, kv_pages, out, scratch, scratch_words, kv_len, n_seqs, max_kv_len, page_table,
                        table_width, n_heads, n_kv, scale, status, s);
}
