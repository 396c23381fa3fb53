// Causal attention of a step's new tokens over the paged cache on the 5th-
// generation tensor cores (tcgen05), bfloat16, head sizes 64 and 128.
//
// A block takes one query head and 128 consecutive new tokens of one sequence
// (two of the step's 64-row work items) and walks over the keys in blocks of 128
// (two cache pages):
//   * a producer thread fetches the query rows once and the key and value pages
//     through a ring of six tiles (TMA, 64 x 64 boxes, 128-byte swizzle); a key
//     tile is free again as soon as its scores are computed;
//   * an issuing thread computes S = Q K^T into one of three 128-column buffers
//     of tensor memory, up to three blocks ahead of the softmax, and accumulates
//     O += P V (the values are the MN-major operand: their rows are keys);
//   * eight warps own one query row per pair of threads (64 keys of a block each;
//     the row's maximum crosses through shared memory): they read S from tensor
//     memory, scale, mask (a key is visible up to the token's own position), and
//     write P as pairs of bfloat16 back into tensor memory over the scores it
//     came from, where the second product takes it from.  With three buffers the
//     softmax of the next block never waits for a product: what bounds a block
//     is the 16 instructions the tensor core takes for it (one every ~93 clocks).
// O and the sum are scaled by a maximum that follows the true running maximum
// lazily: only when a block's maximum exceeds it by more than 8 (in units of
// log2 e) is O rescaled in tensor memory, so that after the first blocks of a row
// the rescaling is rare; probabilities stay below 2^8, which bfloat16 and
// float32 hold without loss of relative precision.
// Value rows beyond the cached length are zeroed in shared memory before they
// are multiplied (their weight is zero, but the row may hold anything).
// Every wait is bounded and reports through the status word.
// Formulas: wick src/model.rs:520-553.  The plain forms of this computation are
// attn_prompt_mma_kernel (attn_prompt_mma.cu) and attn_prompt_kernel (attn.cu).
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"
#include "tcgen05.cuh"

#ifndef WICK_HD
#error "compile with -DWICK_HD=<head_dim>"
#endif

namespace wick {
namespace prompttc {

constexpr bool SUPPORTED = WICK_HD == 64 || WICK_HD == 128;
constexpr int HD = SUPPORTED ? WICK_HD : 64;           // other head sizes: the entry point refuses, the kernel is never launched
constexpr int BQ = 128;                                // query rows of a block
constexpr int BK = 128;                                // keys of an inner step (two pages)
constexpr int PANELS = HD / 64;                        // 64-column panels of a head row
constexpr int PANEL_BYTES = 128 * 128;                 // 128 rows of 128 bytes
constexpr int TILE_BYTES = PANELS * PANEL_BYTES;       // Q, or one block of keys or of values
constexpr int NSLOT = 6;                               // key / value tiles in flight: 2 per score buffer (the ring of
                                                       // tiles and the ring of score buffers turn together)
constexpr int SMEM_BYTES = TILE_BYTES + NSLOT * TILE_BYTES + 1024;
constexpr int THREADS = 320;                           // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-9: softmax
constexpr int NBUF = 3;                                // score buffers
static_assert(NSLOT == 2 * NBUF, "a tile slot is free when the scores (the product) of three blocks before are done");
constexpr int HALF_K = BK / 2;                         // keys of a block that one softmax thread handles
constexpr uint32_t TMEM_COLS = 512;                    // S0 | S1 | S2 | O; P (bfloat16 pairs) takes the place of the
constexpr uint32_t COL_S = 0, COL_O = NBUF * BK;       // first 64 columns of the S buffer it was computed from
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Two barriers at once (their polls overlap).
__device__ __forceinline__ bool mbar_wait2(uint64_t* a, uint32_t pa, uint64_t* b, uint32_t pb, volatile int* abort_flag, int* status, int code) {
    const bool ra = mbar_try_wait(a, pa), rb = mbar_try_wait(b, pb);
    if (ra && rb) return true;
    return (ra || mbar_wait(a, pa, abort_flag, status, code)) && (rb || mbar_wait(b, pb, abort_flag, status, code));
}
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The issuing thread is one thread: what it computes per instruction is what limits
// the rate of small products.  A shared-memory descriptor is therefore kept as two
// 32-bit halves: the high half is a constant, the low half (start address in 16-byte
// units, leading offset) moves by one addition per instruction.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
// stride offset 1024 bytes (8 rows of 128 bytes), descriptor version 1 (bit 46), 128-byte swizzle (bits 61-63)
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);

// D (tensor memory) (+)= A (shared memory) * B (shared memory)
template <int ACC>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "n"(ACC)
        : "memory");
}
// D (tensor memory) (+)= A (tensor memory: 128 lanes x 8 columns of bfloat16 pairs) * B (shared memory)
template <int ACC>
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "n"(ACC)
        : "memory");
}
template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// The softmax warps are bound by the number of instructions they issue: two products-and-sums,
// two sums, or a maximum of three per instruction where sm_100 has one.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {      // a * b + c, each half rounded once
    uint64_t ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    uint64_t ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// Descriptors.  A k-major operand (Q, K): rows of 128 bytes, eight-row groups 1024
// bytes apart, the leading offset unused (1).  The MN-major operand (V): rows are
// keys, a row holds 64 consecutive dims in 128 bytes, eight rows make a 1024-byte
// group, and the next 64 dims lie one panel (the leading offset) further.

__global__ void __launch_bounds__(THREADS, 1)
attn_prompt_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                      bf16* __restrict__ out, const int* __restrict__ cu_seqlens, int n_seqs,
                      const int* __restrict__ start_arr,
                      const int* __restrict__ page_table, int table_width, int n_tiles, int n_heads, int n_kv,
                      float scale, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t q_full, full[NSLOT];
    __shared__ uint64_t s_full[NBUF], p_full[NBUF], pv_done[2], v_free[NBUF], x_bar[4];   // pv_done: even blocks, odd blocks
    __shared__ bf16 mx_x[2][2][BQ];                            // the maxima the two halves of a row tell each other
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    pdl_trigger();
    // longest first: the last work items of a sequence see the most keys
    // (the step's description is written by the host before the step: no kernel produces it)
    int b, q0;
    find_work_item(cu_seqlens, n_seqs, 64, n_tiles - 1 - (int)blockIdx.x, b, q0);
    if (b < 0 || q0 % BQ != 0) return;                             // the odd 64-row item belongs to its even neighbour's block
    const int head = blockIdx.y, kvh = head / (n_heads / n_kv);
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0, start = start_arr[b];
    const int kv_len = start + q_len;
    const int rows = min(BQ, q_len - q0);
    const int last_key = min(start + q0 + BQ - 1, kv_len - 1);     // the last position any row of the block may see
    const int n_blk = last_key / BK + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = base;
    uint8_t* kv_s = q_s + TILE_BYTES;                              // NSLOT tiles: keys and values of the blocks in flight

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&q_full, 1);
        for (int s = 0; s < NSLOT; ++s) mbar_init(&full[s], 1);
        for (int i = 0; i < NBUF; ++i) {
            mbar_init(&s_full[i], 1);
            // One arrival per softmax warp; a barrier per score buffer, since a warp may be up to
            // two blocks ahead of another (never three: the scores of block j + 3 wait for P V of block j).
            mbar_init(&p_full[i], 8);
        }
        mbar_init(&pv_done[0], 1);
        mbar_init(&pv_done[1], 1);
        for (int i = 0; i < NBUF; ++i) mbar_init(&v_free[i], 1);
        for (int i = 0; i < 4; ++i) mbar_init(&x_bar[i], 2);       // the two warps that share 32 rows
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_wait();                                                    // q and the cache come from the kernel before this one

    if (warp == 0) {
        // ---------------- producer ----------------
        // Items in order K_0, V_0, K_1, V_1, ...; item i lives in slot i % NSLOT.
        if (lane == 0) {
            mbar_expect_tx(&q_full, TILE_BYTES);
            for (int pn = 0; pn < PANELS; ++pn) tma_load_2d(&q_map, &q_full, q_s + pn * PANEL_BYTES, head * HD + pn * 64, tok0 + q0);
            for (int i = 0; i < 2 * n_blk; ++i) {
                const int slot = i % NSLOT, j = i >> 1, is_v = i & 1;
                // The slot held the keys (values) of block j - 3: free when that block's scores are
                // computed (its P V product is complete), which is what s_full (v_free) says.  Each
                // of these barriers completes one phase per visit of this thread, and its next phase
                // needs the tile that is fetched after the wait: it can never be two phases on, which
                // a parity could not tell from none.  (pv_done, which alternate blocks share, could:
                // nothing holds the last two products back while this thread is late.)
                if (j >= NBUF) {
                    const int jp = j - NBUF;
                    if (!mbar_wait(is_v ? &v_free[jp % NBUF] : &s_full[jp % NBUF], (jp / NBUF) & 1, &abort_flag, status, 7)) break;
                }
                mbar_expect_tx(&full[slot], TILE_BYTES);
                for (int w = 0; w < 2; ++w) {
                    const int idx = 2 * j + w;
                    const int page = idx < table_width ? page_table[(int64_t)b * table_width + idx] : 0;
                    for (int pn = 0; pn < PANELS; ++pn)
                        tma_load_2d(&kv_map, &full[slot], kv_s + slot * TILE_BYTES + pn * PANEL_BYTES + w * (kPage * 128), pn * 64,
                                    ((page * 2 + is_v) * n_kv + kvh) * kPage);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // Block j: scores in S[j % 3], all blocks accumulate into the one O.
        // (Measured on this part: the tensor core takes an instruction of this kind every
        // ~93 clocks at best, whatever its width up to N = 128; 16 of them make a block.)
        if (lane == 0) {
            // kind::f16, bfloat16 operands, float32 accumulator, M = 128
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BK >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            const uint32_t q_lo = desc_lo(smem_u32(q_s), 16);
            const uint32_t k_lo0 = desc_lo(smem_u32(kv_s), 16), v_lo0 = desc_lo(smem_u32(kv_s), PANEL_BYTES);
            auto issue_s = [&](int j) -> bool {
                const int i = 2 * j, slot = i % NSLOT, buf = j % NBUF;
                if (!mbar_wait(&full[slot], (i / NSLOT) & 1, &abort_flag, status, 7)) return false;
                tc_fence_after();
                const uint32_t k_lo = k_lo0 + slot * (TILE_BYTES >> 4), d = tmem + COL_S + buf * BK;
                static_for<0, HD / 16>([&](auto ks) {
                    constexpr uint32_t off = (((int)ks >> 2) * PANEL_BYTES + ((int)ks & 3) * 32) >> 4;
                    mma_ss<((int)ks > 0)>(d, q_lo + off, k_lo + off, idesc_s);
                });
                tc_commit(&s_full[buf]);                                     // (also: the keys are read)
                return true;
            };
            bool ok = mbar_wait(&q_full, 0, &abort_flag, status, 7);
            for (int j = 0; j < NBUF && j < n_blk && ok; ++j) ok = issue_s(j);
            for (int j = 0; j < n_blk && ok; ++j) {
                const int i = 2 * j + 1, slot = i % NSLOT;
                ok = ok && mbar_wait2(&p_full[j % NBUF], (j / NBUF) & 1, &full[slot], (i / NSLOT) & 1, &abort_flag, status, 7);
                if (!ok) break;
                tc_fence_after();
                const uint32_t v_lo = v_lo0 + slot * (TILE_BYTES >> 4), d = tmem + COL_O, pa = tmem + COL_S + (j % NBUF) * BK;
                if (j > 0) mma_ts<1>(d, pa, v_lo, idesc_o);
                else mma_ts<0>(d, pa, v_lo, idesc_o);
                static_for<1, BK / 16>([&](auto ks) { mma_ts<1>(d, pa + (int)ks * 8, v_lo + (int)ks * (2048 >> 4), idesc_o); });
                tc_commit(&pv_done[j & 1]);
                tc_commit(&v_free[j % NBUF]);                                // the values are read: their tile is free
                if (j + NBUF < n_blk) {
                    // the scores of block j + 3 go where this block's P lies: only when it has been read
                    ok = mbar_wait(&pv_done[j & 1], (j >> 1) & 1, &abort_flag, status, 7) && issue_s(j + NBUF);
                }
            }
        }
    } else {
        // ---------------- softmax: a query row per pair of threads ----------------
        // Warps 2-5 take keys 0-63 of a block, warps 6-9 keys 64-127 of the same rows
        // (a warp reads the 32 lanes of tensor memory given by its index modulo 4).
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int r = quad * 32 + lane;
        const int c_lo = half * HALF_K;
        const int q_pos = start + q0 + r;
        const int limit = min(q_pos, kv_len - 1);                   // last visible key position
        const float sl2 = scale * 1.4426950408889634f;
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        constexpr int OW = HD / 2;                                  // columns of O this thread rescales and stores
        const uint32_t o_addr = lane_base + COL_O + half * OW;
        // m: the maximum (in units of log2 e) that O and l are scaled by.  It follows
        // the true running maximum lazily; l: this thread's part of the row's sum.
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blk; ++j) {
            const int buf = j % NBUF, xb = j & 1, v_item = 2 * j + 1, v_slot = v_item % NSLOT;
            const uint32_t s_addr = lane_base + COL_S + buf * BK;
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[buf], (j / NBUF) & 1, &abort_flag, status, 7));
            if (!ok) break;
            tc_fence_after();
            const int key0 = j * BK + c_lo;
            float s[HALF_K];
            tc_ld32_nowait(s_addr + c_lo, reinterpret_cast<uint32_t*>(s));
            tc_ld32_nowait(s_addr + c_lo + 32, reinterpret_cast<uint32_t*>(s + 32));
            tc_ld_wait();
            if (key0 + HALF_K - 1 > limit) {
#pragma unroll
                for (int i = 0; i < HALF_K; ++i)
                    if (key0 + i > limit) s[i] = -INFINITY;
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < HALF_K; i += 8) {
                mx4[0] = max3(mx4[0], s[i], s[i + 1]);
                mx4[1] = max3(mx4[1], s[i + 2], s[i + 3]);
                mx4[2] = max3(mx4[2], s[i + 4], s[i + 5]);
                mx4[3] = max3(mx4[3], s[i + 6], s[i + 7]);
            }
            // The row's other half: through shared memory and the pair's barrier.  Both sides
            // round to bfloat16, so that both scale by the same number (the scaling maximum
            // need not be the exact one).
            const bf16 mx_mine = __float2bfloat16_rn(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            mx_x[xb][half][r] = mx_mine;
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_bar[quad]);
            ok = __all_sync(0xffffffffu, mbar_wait(&x_bar[quad], j & 1, &abort_flag, status, 7));
            if (!ok) break;
            const float mx = fmaxf(__bfloat162float(mx_mine), __bfloat162float(mx_x[xb][half ^ 1][r])) * sl2;
            const bool grow = mx > m + 8.0f;
            float alpha = 1.0f;
            if (grow) {
                alpha = ex2(m - mx);                                // 0 for the first keys a row sees
                m = mx;
            }
            const float neg_m = m == -INFINITY ? 0.f : -m;          // a row that sees no key yet
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // Rare.  O must hold the product of the block before.  (Its barrier serves every other
                // block; that the scores of this block exist says that the product of block j - 3, the
                // barrier's phase before, is complete: the parity is unambiguous although most blocks
                // never wait here.)
                ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, &abort_flag, status, 7));
                if (!ok) break;
                tc_fence_after();
                {
#pragma unroll
                    for (int c = 0; c < OW; c += 32) {
                        uint32_t raw[32];
                        tc_ld32_nowait(o_addr + c, raw);
                        tc_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
                        tc_st32(o_addr + c, raw);
                    }
                    tc_st_wait();
                }
            }
            float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
            uint32_t packed[HALF_K / 2];
            const float2 sl2_2 = make_float2(sl2, sl2), neg_m2 = make_float2(neg_m, neg_m);
#pragma unroll
            for (int i = 0; i < HALF_K; i += 2) {
                const float2 x = fma2(make_float2(s[i], s[i + 1]), sl2_2, neg_m2);
                const float2 pp = make_float2(ex2(x.x), ex2(x.y));
                sum2[(i >> 1) & 3] = add2(sum2[(i >> 1) & 3], pp);
                __nv_bfloat162 hh = __floats2bfloat162_rn(pp.x, pp.y);      // key 2k in the low half, key 2k + 1 in the high half
                packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
            }
            const float sum4[4] = {sum2[0].x + sum2[0].y, sum2[1].x + sum2[1].y, sum2[2].x + sum2[2].y, sum2[3].x + sum2[3].y};
            // P over the scores it came from (the other half has its scores in registers: it passed the pair's barrier)
            tc_st32(s_addr + half * (HALF_K / 2), packed);
            tc_st_wait();
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            // value rows that hold no token yet are made zero before they are multiplied
            const int valid = kv_len - j * BK;
            if (valid < BK) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full[v_slot], (v_item / NSLOT) & 1, &abort_flag, status, 7));
                if (!ok) break;
                const int first = max(valid, 0);
                for (int i = threadIdx.x - 64; i < (BK - first) * (HD / 8); i += THREADS - 64) {
                    const int row = first + i / (HD / 8), chunk = i % (HD / 8);
                    *reinterpret_cast<uint4*>(kv_s + v_slot * TILE_BYTES + (chunk >> 3) * PANEL_BYTES + row * 128 +
                                              (((chunk & 7) ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros before the tensor core reads them
            }
            tc_fence_before();                                               // P and the rescaled O before it multiplies and accumulates
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[buf]);
        }
        // the last products, in their order (each wait with an unambiguous parity: see above)
        if (ok && n_blk > 1) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(n_blk - 2) & 1], ((n_blk - 2) >> 1) & 1, &abort_flag, status, 7));
        ok = ok && __all_sync(0xffffffffu, mbar_wait(&pv_done[(n_blk - 1) & 1], ((n_blk - 1) >> 1) & 1, &abort_flag, status, 7));
        tc_fence_after();
        float* l_x = reinterpret_cast<float*>(&mx_x[0][0][0]);       // free once every block's maxima have been read
        if (ok) {
            // the row's sum: this half's plus the other's, in a fixed order
            l_x[half * BQ + r] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_bar[quad]);
            ok = __all_sync(0xffffffffu, mbar_wait(&x_bar[quad], n_blk & 1, &abort_flag, status, 7));
        }
        if (ok) {
            // every lane takes part in the loads from tensor memory; only rows that exist are stored
            const float l_row = l_x[r] + l_x[BQ + r];
            const bool store = r < rows && l_row > 0.f;
            const float inv = store ? 1.0f / l_row : 0.f;
            bf16* dst = out + ((int64_t)(tok0 + q0 + r) * n_heads + head) * HD + half * OW;
#pragma unroll
            for (int c = 0; c < OW; c += 32) {
                uint32_t raw[32];
                tc_ld32_nowait(o_addr + c, raw);
                tc_ld_wait();
                if (store) {
#pragma unroll
                    for (int g4 = 0; g4 < 4; ++g4) {
                        uint4 w;
                        __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            hh[i] = __floats2bfloat162_rn(__uint_as_float(raw[8 * g4 + 2 * i]) * inv, __uint_as_float(raw[8 * g4 + 2 * i + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + 8 * g4) = w;
                    }
                }
                __syncwarp();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);   // copies in flight land before the block leaves
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

}  // namespace prompttc
}  // namespace wick

using namespace wick;

WICK_API int wick_attn_prompt_tc_supported() { return prompttc::SUPPORTED ? 1 : 0; }

// q, out: bfloat16 [n_tokens, n_heads, HD]; kv: one schedule entry's cache, bfloat16
// [kv_pages, 2, n_kv, 64, HD] (it already holds the new tokens' keys and values);
// n_tiles: the step's 64-row work items (one per 64 new tokens of a sequence, numbered
// sequence by sequence); status: device int (code 7 if a block gave up waiting).
WICK_API int wick_attn_prompt_tc_bf16(const void* q, long long n_tokens, const void* kv, long long kv_pages, void* out,
                                      int n_tiles, const int* cu_seqlens, int n_seqs,
                                      const int* start, const int* page_table, int table_width, int n_heads, int n_kv,
                                      float scale, int* status, void* s) {
    using namespace prompttc;
    WICK_REQUIRE(SUPPORTED, "attention (tcgen05): head_dim %d is not 64 or 128", (int)WICK_HD);
    WICK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads over %d kv heads", n_heads, n_kv);
    WICK_REQUIRE(n_heads <= 65535, "attention: %d heads is beyond the grid limit", n_heads);
    if (n_tiles == 0) return 0;
    CUtensorMap q_map, kv_map;
    if (int e = make_bf16_map(&q_map, q, n_tokens, (long long)n_heads * HD, BQ, "attention (tcgen05)")) return e;
    if (int e = make_bf16_map(&kv_map, kv, kv_pages * 2 * n_kv * kPage, HD, kPage, "attention (tcgen05)")) return e;
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(attn_prompt_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        raised = true;
    }
    WICK_CUDA(launch(attn_prompt_tc_kernel, dim3(n_tiles, n_heads), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)s, q_map,
                     kv_map, (bf16*)out, cu_seqlens, n_seqs, start, page_table, table_width, n_tiles, n_heads,
                     n_kv, scale, status));
    return check_launch("attn_prompt_tc");
}
