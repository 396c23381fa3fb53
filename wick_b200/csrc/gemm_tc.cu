// D[m, n] = sum_k A[m, k] * B[n, k] for bfloat16 operands that are both
// contiguous along k, on the 5th-generation tensor cores of sm_100a:
//
//   * TMA (cp.async.bulk.tensor, 128-byte swizzle) stages 128 x 64 tiles of A and
//     bn x 64 tiles of B in a ring of shared-memory buffers;
//   * one elected thread issues tcgen05.mma (M = 128, N = bn, K = 16 per
//     instruction) with the float32 accumulator in tensor memory;
//   * four warps read the accumulator back with tcgen05.ld and write the result.
//
// The same kernel serves both shapes of work.  Prompts: A = activations
// [tokens, k], B = weights [out, k], D written row-major [tokens, out].  Decode
// (few tokens): A = weights, B = activations (bn = tokens rounded up to 16), D
// written transposed, so that the 128-row side of the instruction is always
// full and every CTA streams a 128-row slab of the weight matrix.  Options:
// a gated pair (two accumulators, silu(g) * u in the epilogue; wick
// src/model.rs:493-501), float32 or bfloat16 output, and a split of the k range
// over blockIdx.z into float32 partial sums that the consumer adds in index
// order.  Each output element is accumulated along k in index order within a
// split, whatever the tile it falls into, so a row's result does not depend on
// the other rows of the batch.
//
// Every wait on an mbarrier is bounded (about one second); when a wait gives up,
// the kernel records a code in *status, stops waiting anywhere, lets copies in
// flight land, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"
#include "tcgen05.cuh"

namespace wick {

constexpr int BM = 128;            // rows of the A tile = M of the instruction
constexpr int BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 12;
constexpr int NUM_THREADS = 192;   // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

struct GemmParams {
    int a_rows;                    // valid rows of A (outputs beyond are not written)
    int b_rows;                    // valid rows of B
    int bn;                        // rows of a B tile = N of the instruction (multiple of 16, <= 256)
    int k_blocks;                  // ceil(k / 64)
    int k_blocks_per_split;
    int stages;
    int gated;                     // 0 none, 1 the pair lives in A (two tiles), 2 the pair lives in B (two tiles),
                                   // 3 the pair lives in A and shares one tile: rows 0-63 gate, rows 64-127 up
    int pair_offset;               // row offset of the second half of the pair
    int transposed;                // 0: out[m * ldo + n], 1: out[n * ldo + m]
    int out_f32;
    int total_tiles, grid_m, grid_n;   // tiles = grid_m * grid_n * splits, the m tile varying fastest
    int a_packed, b_packed;        // that operand is stored as tiles of 128 rows x 64 columns (see wick_gemm_tc)
    int a_static;                  // A is never written by a kernel (weights): it may be fetched before the
    int b_static;                  //   preceding kernel has finished; likewise B
    long long ldo;
    long long split_stride;        // elements between the partial results of two splits
    void* out;
    int* status;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent: block b works on tiles b, b + gridDim.x, ...  A tile is (m tile, n
// tile, split) with the m tile varying fastest, so that blocks running at the
// same time share B tiles through the L2 cache.  With two accumulators in tensor
// memory the epilogue of one tile overlaps the main loop of the next.
template <bool PERSIST, int GATED, bool TRANSPOSED, bool OUT_F32>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[MAX_STAGES];
    __shared__ uint64_t empty_bar[MAX_STAGES];
    __shared__ uint64_t acc_full[2];
    __shared__ uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int ok_w[4];
    __shared__ float xch[2][64][17];           // gated == 3: up values on their way to the warps that hold the gate values

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = GATED == 3 ? BM / 2 : BM;
    const int a_tiles = GATED == 1 ? 2 : 1, b_tiles = GATED == 2 ? 2 : 1;
    const uint32_t a_bytes = BM * BK * 2, b_bytes = (uint32_t)p.bn * BK * 2;
    const uint32_t stage_bytes = a_tiles * a_bytes + b_tiles * b_bytes;
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int n_acc = (GATED == 1 || GATED == 2) ? 2 : 1;
    const int acc_cols = n_acc * p.bn;                       // columns of one tile's accumulators
    // PERSIST: block b runs tiles b, b + gridDim.x, ...; otherwise the grid is (m tiles, n tiles, splits).
    const int my_tiles = PERSIST ? (p.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 1;
    const int w_first = PERSIST ? (int)blockIdx.x : 0, w_end = PERSIST ? p.total_tiles : 1;
    const int w_step = PERSIST ? (int)gridDim.x : 1;
    const int acc_bufs = (my_tiles > 1 && 2 * acc_cols <= 512) ? 2 : 1;
    uint32_t tmem_cols = 32;
    while (tmem_cols < (uint32_t)(acc_bufs * acc_cols)) tmem_cols <<= 1;

    auto tile_coords = [&](int w, int& m0, int& n0, int& kb_begin, int& n_kb, int& z) {
        int x, y;
        if (PERSIST) {
            x = w % p.grid_m;
            y = (w / p.grid_m) % p.grid_n;
            z = w / (p.grid_m * p.grid_n);
        } else {                                             // one tile per block: a three-dimensional grid
            x = blockIdx.x;
            y = blockIdx.y;
            z = blockIdx.z;
        }
        m0 = x * tile_m;
        n0 = y * p.bn;
        kb_begin = z * p.k_blocks_per_split;
        n_kb = min(p.k_blocks, kb_begin + p.k_blocks_per_split) - kb_begin;
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);                     // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;                                 // 64-wide steps issued so far, over all tiles
            bool ok = true;
            for (int w = w_first; w < w_end && ok; w += w_step) {
                int m0, n0, kb_begin, n_kb, z;
                tile_coords(w, m0, n0, kb_begin, n_kb, z);
                // Coordinates of the box that holds rows row.. of k-block kb: in a row-major
                // operand (kb * 64, row); in a packed one the tile (row / 128, kb) lies as
                // 128 contiguous lines of 128 bytes.
                auto load = [&](const CUtensorMap* map, int packed, int s, void* dst, int kb, int row) {
                    if (packed) tma_load_2d(map, &full_bar[s], dst, 0, ((row >> 7) * p.k_blocks + kb) * 128 + (row & 127));
                    else tma_load_2d(map, &full_bar[s], dst, kb * BK, row);
                };
                auto load_a = [&](int i, int s) {
                    uint8_t* st = tiles + (size_t)s * stage_bytes;
                    const int kb = kb_begin + i;
                    load(&map_a, p.a_packed, s, st, kb, m0);
                    if (a_tiles == 2) load(&map_a, p.a_packed, s, st + a_bytes, kb, m0 + p.pair_offset);
                    if (GATED == 3) load(&map_a, p.a_packed, s, st + a_bytes / 2, kb, m0 + p.pair_offset);   // 64-row boxes
                };
                auto load_b = [&](int i, int s) {
                    uint8_t* sb = tiles + (size_t)s * stage_bytes + a_tiles * a_bytes;
                    const int kb = kb_begin + i;
                    load(&map_b, p.b_packed, s, sb, kb, n0);
                    if (p.b_packed && p.bn > 128) load(&map_b, p.b_packed, s, sb + 128 * BK * 2, kb, n0 + 128);   // 256 rows: two tiles
                    if (b_tiles == 2) load(&map_b, p.b_packed, s, sb + b_bytes, kb, n0 + p.pair_offset);
                };
                int i = 0;
                if (it == 0) {
                    // The first ring of stages is free.  An operand that no kernel
                    // writes (weights) is fetched before the preceding kernel has
                    // finished; the other one only after pdl_wait.
                    const int first = min(n_kb, p.stages);
                    for (int j = 0; j < first; ++j) {
                        mbar_expect_tx(&full_bar[j], stage_bytes);
                        if (p.a_static) load_a(j, j);
                        if (p.b_static) load_b(j, j);
                    }
                    pdl_wait();
                    for (int j = 0; j < first; ++j) {
                        if (!p.a_static) load_a(j, j);
                        if (!p.b_static) load_b(j, j);
                    }
                    i = first;
                    it = first;
                }
                for (; i < n_kb; ++i, ++it) {
                    const int s = it % p.stages;
                    const uint32_t round = it / p.stages;
                    if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &abort_flag, p.status, 1)) { ok = false; break; }
                    mbar_expect_tx(&full_bar[s], stage_bytes);
                    load_a(i, s);
                    load_b(i, s);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // kind::f16, A and B bfloat16 and k-major, float32 accumulator, M = 128, N = bn
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0;
            bool ok = true;
            int t = 0;
            for (int w = w_first; w < w_end && ok; w += w_step, ++t) {
                int m0, n0, kb_begin, n_kb, z;
                tile_coords(w, m0, n0, kb_begin, n_kb, z);
                const int buf = acc_bufs == 2 ? (t & 1) : 0;
                const uint32_t use = acc_bufs == 2 ? (uint32_t)(t >> 1) : (uint32_t)t;   // how often this buffer was used before
                if (t > 0) {
                    ok = mbar_wait(&acc_empty[buf], (use & 1) ^ 1, &abort_flag, p.status, 5);  // the epilogue has drained it
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d0 = tmem_base + buf * acc_cols;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % p.stages;
                    const uint32_t round = it / p.stages;
                    ok = mbar_wait(&full_bar[s], round & 1, &abort_flag, p.status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(tiles + (size_t)s * stage_bytes);
                    const uint32_t sb = sa + a_tiles * a_bytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                        const uint64_t da = smem_desc(sa + k * UMMA_K * 2), db = smem_desc(sb + k * UMMA_K * 2);
                        tc_mma(d0, da, db, idesc, acc);
                        if (GATED == 1) tc_mma(d0 + p.bn, smem_desc(sa + a_bytes + k * UMMA_K * 2), db, idesc, acc);
                        if (GATED == 2) tc_mma(d0 + p.bn, da, smem_desc(sb + b_bytes + k * UMMA_K * 2), idesc, acc);
                    }
                    tc_commit(&empty_bar[s]);      // the stage is free once these instructions have read it
                }
                tc_commit(&acc_full[buf]);         // this tile's accumulator is complete
            }
        }
    } else {
        // ---------------- epilogue: tensor memory -> global ----------------
        const int q = warp & 3;                    // this warp reads lanes 32q .. 32q+31
        pdl_wait();                                // the output may alias memory an earlier kernel still reads
        int t = 0;
        for (int w = w_first; w < w_end; w += w_step, ++t) {
            int m0, n0, kb_begin, n_kb, z;
            tile_coords(w, m0, n0, kb_begin, n_kb, z);
            const int buf = acc_bufs == 2 ? (t & 1) : 0;
            const uint32_t use = acc_bufs == 2 ? (uint32_t)(t >> 1) : (uint32_t)t;
            const int m = m0 + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + buf * acc_cols + ((uint32_t)(q * 32) << 16);
            char* out_base = (char*)p.out + (size_t)z * p.split_stride * (OUT_F32 ? 4 : 2);
            // One answer for the four epilogue warps, so that they leave the loop together.
            const bool ok_warp = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], use & 1, &abort_flag, p.status, 3));
            bool ok = ok_warp;
            if (my_tiles > 1 || GATED == 3) {            // (a block with one plain tile has nothing left to agree on)
                if (lane == 0) ok_w[q] = ok_warp ? 1 : 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                ok = ok_w[0] && ok_w[1] && ok_w[2] && ok_w[3];
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            tc_fence_after();
            if (GATED == 3) {
                // Lanes 0-63 of the accumulator hold gate rows, lanes 64-127 the up rows of the
                // same outputs (transposed output only).  Of every 16 columns the warps of the gate
                // rows finish and store the first 8, the warps of the up rows the last 8 (the
                // activation's exponential and division are the long part of a decode block's
                // end: all four warps share them); what each side lacks crosses through shared
                // memory.
                const int mg = m0 + (q & 1) * 32 + lane, xrow = (q & 1) * 32 + lane;
                const bool upper = q >= 2;
                for (int c0 = 0; c0 < p.bn; c0 += 16) {
                    float v[16];
                    if (ok && n_kb > 0) tc_ld16(lane_addr + c0, v);
                    float (*xb)[17] = xch[(c0 >> 4) & 1];
#pragma unroll
                    for (int j = 0; j < 8; ++j) xb[xrow][upper ? j : 8 + j] = upper ? v[j] : v[8 + j];
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (ok && n_kb > 0 && mg < p.a_rows) {
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) {
                            const int j = upper ? 8 + jj : jj;
                            const int n = n0 + c0 + j;
                            if (n < p.b_rows) {
                                const float mine = upper ? v[8 + jj] : v[jj], other = xb[xrow][j];
                                const float g = upper ? other : mine, u = upper ? mine : other;
                                const float r = g / (1.0f + expf(-g)) * u;
                                const long long off = (long long)n * p.ldo + mg;
                                if (OUT_F32) ((float*)out_base)[off] = r;
                                else ((__nv_bfloat16*)out_base)[off] = __float2bfloat16_rn(r);
                            }
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");     // the exchange buffers are free for the next tile
            } else if (ok && n_kb > 0) {
                for (int c0 = 0; c0 < p.bn; c0 += 16) {
                    float v[16];
                    tc_ld16(lane_addr + c0, v);
                    if (GATED) {
                        float u[16];
                        tc_ld16(lane_addr + p.bn + c0, u);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = v[j] / (1.0f + expf(-v[j])) * u[j];
                    }
                    if (m < p.a_rows) {
                        if (!TRANSPOSED) {
                            const int n_left = p.b_rows - (n0 + c0);
                            const long long off = (long long)m * p.ldo + n0 + c0;
                            if (OUT_F32) {
                                float* o = (float*)out_base + off;
                                if (n_left >= 16 && (off & 3) == 0) {
#pragma unroll
                                    for (int j = 0; j < 16; j += 4) *(float4*)(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                } else {
                                    for (int j = 0; j < 16 && j < n_left; ++j) o[j] = v[j];
                                }
                            } else {
                                __nv_bfloat16* o = (__nv_bfloat16*)out_base + off;
                                if (n_left >= 16 && (off & 7) == 0) {
                                    uint4 wv[2];
                                    __nv_bfloat162* h = (__nv_bfloat162*)wv;
#pragma unroll
                                    for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                    *(uint4*)o = wv[0];
                                    *(uint4*)(o + 8) = wv[1];
                                } else {
                                    for (int j = 0; j < 16 && j < n_left; ++j) o[j] = __float2bfloat16_rn(v[j]);
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int n = n0 + c0 + j;
                                if (n < p.b_rows) {
                                    const long long off = (long long)n * p.ldo + m;
                                    if (OUT_F32) ((float*)out_base)[off] = v[j];
                                    else ((__nv_bfloat16*)out_base)[off] = __float2bfloat16_rn(v[j]);
                                }
                            }
                        }
                    }
                }
            }
            // this warp has read what it needs of the accumulator: hand the buffer back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (!ok) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // Copies that were already issued may still be in flight: give them time
        // to land before this block's shared memory is given up.
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

// ---- host side ---------------------------------------------------------------
// A [rows, k] bfloat16 matrix, row-major, as a TMA descriptor with boxes of box_rows x 64.
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t k, int box_rows) {
    return make_bf16_map(map, ptr, rows, k, box_rows, "gemm_tc");
}

}  // namespace wick

using namespace wick;

// a: [a_total_rows, k] bf16 (the 128-row side), b: [b_total_rows, k] bf16.
// a_rows / b_rows: rows that produce output (for a gated pair: rows of ONE half;
// the other half starts pair_offset rows further).
// gated: 0 none, 1 pair in a, 2 pair in b.  transposed: out[n * ldo + m].
// splits > 1 needs out_f32; partial s lies split_stride elements after s - 1.
// a_static / b_static: that operand is never written by any kernel (weights), so
// the kernel may fetch it before the kernel launched before it has finished.
// a_packed / b_packed: that operand is not row-major but stored as [rows / 128][ceil(k / 64)]
// tiles of 128 rows x 64 columns, each tile contiguous (16 KB), rows and columns padded
// with zeros (a gated pair: each half padded on its own, pair_offset counts padded rows);
// a_total_rows / b_total_rows then count padded rows.  A weight tile then comes from DRAM as
// one contiguous piece instead of 128 pieces of 128 bytes.
// status: device int that receives a non-zero code if a wait inside the kernel gave up.
WICK_API int wick_gemm_tc(const void* a, long long a_total_rows, int a_rows, const void* b, long long b_total_rows,
                          int b_rows, int k, int bn, int gated, int pair_offset, int transposed, int out_f32,
                          int a_static, int b_static, int a_packed, int b_packed, void* out, long long ldo, int splits, long long split_stride, int max_smem_bytes, int* status,
                          void* stream) {
    WICK_REQUIRE(bn % 16 == 0 && bn >= 16 && bn <= 256, "gemm_tc: tile width %d must be a multiple of 16 in [16, 256]", bn);
    WICK_REQUIRE(!(gated == 2 && bn > 128) , "gemm_tc: a gated pair needs two accumulators: tile width <= 128");
    WICK_REQUIRE(gated >= 0 && gated <= 3 && splits >= 1, "gemm_tc: bad options");
    WICK_REQUIRE(gated != 3 || transposed, "gemm_tc: the shared-tile pair is built for the transposed output only");
    WICK_REQUIRE(gated != 1 || transposed, "gemm_tc: a pair in the 128-row operand goes with the transposed output");
    WICK_REQUIRE(gated != 2 || !transposed, "gemm_tc: a pair in the narrow operand goes with the row-major output");
    WICK_REQUIRE(splits == 1 || (out_f32 && !gated), "gemm_tc: a split inner dimension needs plain float32 partial sums");
    WICK_REQUIRE(a_rows > 0 && b_rows >= 0 && k > 0, "gemm_tc: bad sizes");
    if (b_rows == 0) return 0;
    const int k_blocks = ceil_div(k, BK);
    WICK_REQUIRE(splits <= k_blocks, "gemm_tc: %d splits over %d blocks of the inner dimension", splits, k_blocks);
    const int per_split = ceil_div(k_blocks, splits);
    WICK_REQUIRE((long long)(splits - 1) * per_split < k_blocks, "gemm_tc: a split would be empty");
    CUtensorMap map_a, map_b;
    WICK_REQUIRE(!a_packed || a_total_rows % 128 == 0, "gemm_tc: a packed operand has a multiple of 128 rows");
    WICK_REQUIRE(!b_packed || (b_total_rows % 128 == 0 && (bn <= 128 || bn == 256)), "gemm_tc: a packed narrow operand comes in tiles of 128 rows");
    if (int e = a_packed ? make_map(&map_a, a, a_total_rows * k_blocks, 64, gated == 3 ? BM / 2 : BM)
                         : make_map(&map_a, a, a_total_rows, k, gated == 3 ? BM / 2 : BM)) return e;
    if (int e = b_packed ? make_map(&map_b, b, b_total_rows * k_blocks, 64, bn < 128 ? bn : 128)
                         : make_map(&map_b, b, b_total_rows, k, bn)) return e;
    const int stage_bytes = (gated == 1 ? 2 : 1) * BM * BK * 2 + (gated == 2 ? 2 : 1) * bn * BK * 2;
    int budget = max_smem_bytes > 0 ? max_smem_bytes : 200 * 1024;
    if (budget > 208 * 1024) budget = 208 * 1024;     // 227 KB per block minus the static arrays
    int stages = (budget - 1024) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > per_split) stages = per_split < 2 ? 2 : per_split;
    WICK_REQUIRE(stages >= 2, "gemm_tc: %d bytes of shared memory hold fewer than two stages of %d bytes", budget, stage_bytes);
    const int smem = stages * stage_bytes + 1024;
    GemmParams p;
    p.a_rows = a_rows; p.b_rows = b_rows; p.bn = bn; p.k_blocks = k_blocks; p.k_blocks_per_split = per_split;
    p.stages = stages; p.gated = gated; p.pair_offset = pair_offset; p.transposed = transposed; p.out_f32 = out_f32;
    p.ldo = ldo; p.split_stride = split_stride; p.out = out; p.status = status;
    p.a_static = a_static; p.b_static = b_static; p.a_packed = a_packed; p.b_packed = b_packed;
    p.grid_m = ceil_div(a_rows, gated == 3 ? BM / 2 : BM);
    p.grid_n = ceil_div(b_rows, bn);
    const long long total = (long long)p.grid_m * p.grid_n * splits;
    WICK_REQUIRE(total < (1ll << 30), "gemm_tc: too many tiles");
    p.total_tiles = (int)total;
    // persistent blocks: as many as can be resident at once (one or two per SM by shared memory)
    const int resident = sm_count() * ((smem + 12 * 1024) * 2 <= 227 * 1024 ? 2 : 1);
    // Decode orientation (and anything that fits at once): one tile per block, so
    // that a block starting while others still stream overlaps their drain.
    // Prompt orientation with more tiles than resident blocks: persistent blocks.
    const bool persistent = !transposed && p.total_tiles > resident;
    WICK_REQUIRE(persistent || (p.grid_n <= 65535 && splits <= 65535), "gemm_tc: grid limit");
    const dim3 grid = persistent ? dim3(resident) : dim3(p.grid_m, p.grid_n, splits);
    // One instantiation per (persistent, pair mode, orientation, output type): a
    // block of a decode step runs for a few microseconds, so the kernel it loads
    // should hold nothing but its own path.
#define WICK_GEMM_CASE(P, G, T, F)                                                                              \
    if (persistent == P && gated == G && (transposed != 0) == T && (out_f32 != 0) == F) {                       \
        static bool raised_##P##G##T##F = false;                                                                 \
        if (!raised_##P##G##T##F) {                                                                              \
            WICK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<P, G, T, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           210 * 1024));                                                         \
            raised_##P##G##T##F = true;                                                                          \
        }                                                                                                        \
        WICK_CUDA(launch(gemm_tc_kernel<P, G, T, F>, grid, dim3(NUM_THREADS), (size_t)smem, (cudaStream_t)stream, \
                         map_a, map_b, p));                                                                      \
        return check_launch("gemm_tc");                                                                          \
    }
    WICK_GEMM_CASE(false, 0, true, true) WICK_GEMM_CASE(false, 0, true, false)
    WICK_GEMM_CASE(false, 1, true, true) WICK_GEMM_CASE(false, 1, true, false)
    WICK_GEMM_CASE(false, 3, true, true) WICK_GEMM_CASE(false, 3, true, false)
    WICK_GEMM_CASE(false, 0, false, true) WICK_GEMM_CASE(false, 0, false, false)
    WICK_GEMM_CASE(false, 2, false, true) WICK_GEMM_CASE(false, 2, false, false)
    WICK_GEMM_CASE(true, 0, false, true) WICK_GEMM_CASE(true, 0, false, false)
    WICK_GEMM_CASE(true, 2, false, true) WICK_GEMM_CASE(true, 2, false, false)
#undef WICK_GEMM_CASE
    return fail("gemm_tc: no kernel for pair mode %d with %s output", gated, transposed ? "transposed" : "row-major");
}
