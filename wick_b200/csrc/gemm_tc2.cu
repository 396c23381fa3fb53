// D[m, n] = sum_k A[m, k] * B[n, k] for many rows of A (prompts): the matrix
// product of gemm_tc.cu with pairs of thread blocks (tcgen05 cta_group::2).
//
// A pair (a cluster of two blocks on neighbouring SMs) computes a 256 x 256 tile.
// Block r of the pair loads rows [128 r, 128 r + 128) of the A tile and rows
// [128 r, 128 r + 128) of the B tile with plain (non-multicast) TMA copies, and
// holds rows [128 r, ...) of the accumulator in its own tensor memory; the MMA
// instruction, issued by block 0 only, reads both blocks' shared memory.  Per
// 64-wide step each block therefore fetches 32 KB for the work that needs 48 KB
// with single blocks, and six stages fit where four did: the main loop stops
// waiting for the L2 cache.  A gated pair of matrices puts 128 gate rows into
// block 0's half of B and the 128 up rows of the same outputs into block 1's, so
// that columns j and 128 + j of the accumulator meet in the epilogue
// (silu(g) * u; wick src/model.rs:493-501).
//
// Persistent: pair p works on tiles p, p + pairs, ...; two accumulators in tensor
// memory let the epilogue of one tile overlap the main loop of the next.
// With few tiles (a few hundred tokens times a narrow matrix) the inner dimension
// can be cut into `splits` runs: a unit of work is then (tile, run), and run r
// writes its float32 partial sums to out + r * split_stride for the consumer to
// add up in index order (as the decode products of gemm_tc.cu do).
// Barriers: "full" (data of both blocks has landed) lives in block 0; "empty"
// and "accumulator full" exist in both blocks and are signalled by
// tcgen05.commit to both; "accumulator empty" lives in block 0 and collects the
// epilogue warps of both blocks.  Every wait is bounded as in gemm_tc.cu.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"
#include "tcgen05.cuh"

namespace wick {
namespace pair {

constexpr int BM = 128;            // rows of A per block (256 per pair)
constexpr int BNH = 128;           // rows of B per block (256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int STAGE_BYTES = (BM + BNH) * BK * 2;      // 32 KB
constexpr int NUM_THREADS = 192;                       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;            // clears the bit that tells the two blocks' shared memories apart

struct Params {
    int a_rows, b_rows;            // valid rows of A; outputs per row (for a gated pair: of ONE half)
    int k_blocks;
    int b_packed;                  // B is stored as contiguous tiles of 128 rows x 64 columns (see wick_gemm_tc)
    int gated;                     // 0 plain, 1 gate rows in block 0's B half and up rows in block 1's
    int pair_offset;               // row offset of the up half inside B
    int out_f32;
    int grid_m, grid_n, total_tiles;
    int splits;                    // runs of the inner dimension (1: whole)
    long long split_stride;        // elements between the outputs of two runs
    long long ldo;
    void* out;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in block `rank` of the pair.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// TMA load whose bytes are counted on block 0's barrier (same offset), whichever block issues it.
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerMask), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives (once the MMAs issued so far are complete) on the barrier at this offset in both blocks.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int GATED, bool OUT_F32, bool ACC>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES];      // used in block 0: both blocks' copies of a stage have landed
    __shared__ uint64_t empty_bar[STAGES];     // in each block: the MMAs have read the stage
    __shared__ uint64_t acc_full[2];           // in each block: a tile's accumulator is complete
    __shared__ uint64_t acc_empty[2];          // used in block 0: both blocks' epilogues have drained it
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int ok_w[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t tmem_cols = 512;            // two accumulators of 256 columns

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 8);       // four epilogue warps in each of the two blocks
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                            // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_trigger();

    // unit w = run * tiles + tile: the runs of a tile go to different pairs at the same time
    const int total_units = p.total_tiles * p.splits;
    auto tile_coords = [&](int w, int& m0, int& n0) {
        const int tile = w % p.total_tiles;
        const int x = tile % p.grid_m, y = tile / p.grid_m;
        m0 = x * 2 * BM;
        n0 = y * (GATED ? BNH : BN);
    };
    auto k_range = [&](int w, int& k0, int& k1) {
        const int run = w / p.total_tiles;
        k0 = (int)((long long)p.k_blocks * run / p.splits);
        k1 = (int)((long long)p.k_blocks * (run + 1) / p.splits);
    };

    if (warp == 0) {
        // ---------------- TMA producer (in both blocks) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            bool first = true;
            for (int w = pair_id; w < total_units && ok; w += n_pairs) {
                int m0, n0, k0, k1;
                tile_coords(w, m0, n0);
                k_range(w, k0, k1);
                const int a_row = m0 + rank * BM;
                const int b_row = GATED ? (rank == 0 ? n0 : p.pair_offset + n0) : n0 + rank * BNH;
                for (int i = k0; i < k1; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &abort_flag, p.status, 1)) { ok = false; break; }
                    uint8_t* st = tiles + (size_t)s * STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
                    if (p.b_packed) tma_load_2d_pair(&map_b, &full_bar[s], st + BM * BK * 2, 0, ((b_row >> 7) * p.k_blocks + i) * 128);
                    else tma_load_2d_pair(&map_b, &full_bar[s], st + BM * BK * 2, i * BK, b_row);   // weights: no kernel writes them
                    if (first) { pdl_wait(); first = false; }                                  // activations: after the producer of A
                    tma_load_2d_pair(&map_a, &full_bar[s], st, i * BK, a_row);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (block 0 only) ----------------
        if (lane == 0 && rank == 0) {
            // kind::f16, A and B bfloat16 and k-major, float32 accumulator, M = 256 (pair), N = 256
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            uint32_t it = 0;
            bool ok = true;
            int t = 0;
            for (int w = pair_id; w < total_units && ok; w += n_pairs, ++t) {
                int k0, k1;
                k_range(w, k0, k1);
                const int buf = t & 1;
                const uint32_t use = (uint32_t)(t >> 1);
                if (t > 1) {
                    ok = mbar_wait(&acc_empty[buf], (use & 1) ^ 1, &abort_flag, p.status, 5);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d0 = tmem_base + buf * BN;
                for (int i = k0; i < k1; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    ok = mbar_wait(&full_bar[s], round & 1, &abort_flag, p.status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                    const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_pair(d0, smem_desc(sa + k * UMMA_K * 2), smem_desc(sb + k * UMMA_K * 2), idesc, (i > k0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(&empty_bar[s]);     // the stage is free in both blocks
                }
                tc_commit_pair(&acc_full[buf]);        // the tile's accumulator is complete in both blocks
            }
        }
    } else {
        // ---------------- epilogue (in both blocks): tensor memory -> global ----------------
        const int q = warp & 3;
        pdl_wait();
        int t = 0;
        for (int w = pair_id; w < total_units; w += n_pairs, ++t) {
            int m0, n0;
            tile_coords(w, m0, n0);
            const long long run_off = (long long)(w / p.total_tiles) * p.split_stride;
            const int buf = t & 1;
            const uint32_t use = (uint32_t)(t >> 1);
            const int m = m0 + rank * BM + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
            const bool ok_warp = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], use & 1, &abort_flag, p.status, 3));
            if (lane == 0) ok_w[q] = ok_warp ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const bool ok = ok_w[0] && ok_w[1] && ok_w[2] && ok_w[3];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            tc_fence_after();
            if (ok) {
                constexpr int OUT_COLS = GATED ? BNH : BN;
                for (int c0 = 0; c0 < OUT_COLS; c0 += 16) {
                    float v[16];
                    tc_ld16(lane_addr + c0, v);
                    if (GATED) {
                        float u[16];
                        tc_ld16(lane_addr + BNH + c0, u);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = v[j] / (1.0f + expf(-v[j])) * u[j];
                    }
                    if (m < p.a_rows) {
                        const int n_left = p.b_rows - (n0 + c0);
                        const long long off = run_off + (long long)m * p.ldo + n0 + c0;
                        if (OUT_F32) {
                            float* o = (float*)p.out + off;
                            if (n_left >= 16 && (off & 3) == 0) {
                                if (ACC) {                      // out += product: the residual stream takes the result directly
                                    float4 r[4];
#pragma unroll
                                    for (int j = 0; j < 4; ++j) r[j] = *(const float4*)(o + 4 * j);
#pragma unroll
                                    for (int j = 0; j < 4; ++j) { v[4 * j] += r[j].x; v[4 * j + 1] += r[j].y; v[4 * j + 2] += r[j].z; v[4 * j + 3] += r[j].w; }
                                }
#pragma unroll
                                for (int j = 0; j < 16; j += 4) *(float4*)(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            } else {
                                for (int j = 0; j < 16 && j < n_left; ++j) o[j] = ACC ? o[j] + v[j] : v[j];
                            }
                        } else {
                            __nv_bfloat16* o = (__nv_bfloat16*)p.out + off;
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
                    }
                }
            }
            // this warp has read what it needs of the accumulator: tell block 0
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(&acc_empty[buf], 0);
            if (!ok) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync();                            // neither block leaves while the other may still read its shared memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

template <int GATED, bool OUT_F32, bool ACC>
static int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p, int blocks, size_t smem,
                       cudaStream_t stream) {
    static bool raised = false;
    if (!raised) {
        WICK_CUDA(cudaFuncSetAttribute(gemm_tc2_kernel<GATED, OUT_F32, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        raised = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    WICK_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<GATED, OUT_F32, ACC>, map_a, map_b, p));
    return check_launch("gemm_tc2");
}

}  // namespace pair
}  // namespace wick

using namespace wick;

// a: activations [a_rows, k] bf16; b: weights [b_total_rows, k] bf16; out[m * ldo + n], n < b_rows.
// gated: b holds gate rows [0, b_rows) and up rows [pair_offset, pair_offset + b_rows); the
// output is silu(a gate^T) * (a up^T).  accumulate (plain float32 output only): out += the product
// (every element by one thread: no atomics).  b_packed: b in the tiled form described at wick_gemm_tc.
// splits > 1 (plain float32 output without accumulation): run r of the inner dimension writes its
// partial sums to out + r * split_stride.  status as in wick_gemm_tc.
WICK_API int wick_gemm_tc2(const void* a, int a_rows, const void* b, long long b_total_rows, int b_rows, int k, int gated,
                           int pair_offset, int out_f32, int accumulate, int b_packed, void* out, long long ldo, int splits,
                           long long split_stride, int* status, void* stream) {
    using namespace pair;
    WICK_REQUIRE(a_rows > 0 && b_rows > 0 && k > 0, "gemm_tc2: bad sizes");
    WICK_REQUIRE(gated == 0 || gated == 1, "gemm_tc2: bad options");
    WICK_REQUIRE(!accumulate || (out_f32 && !gated), "gemm_tc2: accumulation goes with a plain float32 output");
    WICK_REQUIRE(splits >= 1 && (splits == 1 || (out_f32 && !gated && !accumulate)), "gemm_tc2: partial sums are plain float32 outputs");
    WICK_REQUIRE(splits <= ceil_div(k, BK), "gemm_tc2: %d runs of %d steps", splits, ceil_div(k, BK));
    CUtensorMap map_a, map_b;
    if (int e = make_bf16_map(&map_a, a, a_rows, k, BM, "gemm_tc2")) return e;
    WICK_REQUIRE(!b_packed || (b_total_rows % 128 == 0 && pair_offset % 128 == 0), "gemm_tc2: a packed operand comes in tiles of 128 rows");
    if (int e = b_packed ? make_bf16_map(&map_b, b, b_total_rows * ceil_div(k, BK), 64, BNH, "gemm_tc2")
                         : make_bf16_map(&map_b, b, b_total_rows, k, BNH, "gemm_tc2")) return e;
    Params p;
    p.a_rows = a_rows; p.b_rows = b_rows; p.k_blocks = ceil_div(k, BK); p.gated = gated; p.pair_offset = pair_offset;
    p.out_f32 = out_f32; p.ldo = ldo; p.out = out; p.status = status; p.b_packed = b_packed;
    p.grid_m = ceil_div(a_rows, 2 * BM);
    p.grid_n = ceil_div(b_rows, gated ? BNH : BN);
    const long long total = (long long)p.grid_m * p.grid_n;
    WICK_REQUIRE(total < (1ll << 30), "gemm_tc2: too many tiles");
    p.total_tiles = (int)total;
    p.splits = splits;
    p.split_stride = split_stride;
    WICK_REQUIRE(total * splits < (1ll << 30), "gemm_tc2: too many units");
    const int units = p.total_tiles * splits;
    const int sm_pairs = sm_count() / 2;
    const int pairs = units < sm_pairs ? units : sm_pairs;             // a pair of thread blocks per pair of SMs
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    if (gated) return out_f32 ? launch_pair<1, true, false>(map_a, map_b, p, 2 * pairs, smem, (cudaStream_t)stream)
                              : launch_pair<1, false, false>(map_a, map_b, p, 2 * pairs, smem, (cudaStream_t)stream);
    if (accumulate) return launch_pair<0, true, true>(map_a, map_b, p, 2 * pairs, smem, (cudaStream_t)stream);
    return out_f32 ? launch_pair<0, true, false>(map_a, map_b, p, 2 * pairs, smem, (cudaStream_t)stream)
                   : launch_pair<0, false, false>(map_a, map_b, p, 2 * pairs, smem, (cudaStream_t)stream);
}
