// Turning rows of float32 logits into tokens or candidates: argmax (first
// maximum, wick src/sampler.rs:129-137), a draw from softmax(logits / T)
// (sampler.rs:95-125 without the candidate cuts), and the k largest entries in
// sorted order (sampler.rs:87-94), from which the host applies min-p, top-p and
// the draw exactly as the reference does.  One block of 1024 threads per row;
// every reduction and scan has a fixed order, so a row's result depends on that
// row alone.
#include <limits.h>

#include "common.cuh"

namespace wick {

constexpr int ST = 1024;

__global__ void __launch_bounds__(ST) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_wait();
    logits = fresh(logits);
    const float* x = logits + (int64_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = INT_MAX;
    for (int i = threadIdx.x; i < vocab; i += ST) {
        const float v = x[i];
        if (v > best) { best = v; idx = i; }
    }
    auto better = [](float a, int ia, float b, int ib) { return a > b || (a == b && ia < ib); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x];
        idx = si[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        // Nothing compares greater than a NaN in front, and nothing than -inf everywhere.
        if (threadIdx.x == 0) out[blockIdx.x] = (idx == INT_MAX || x[0] != x[0]) ? 0 : idx;
    }
}

// Inclusive scan over the block's ST values in thread order; returns this
// thread's inclusive value, *total gets the sum.
__device__ __forceinline__ float block_scan(float v, float* warp_tot, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float u = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += u;
        }
        warp_tot[lane] = t;
    }
    __syncthreads();
    if (warp > 0) v += warp_tot[warp - 1];
    *total = warp_tot[31];
    return v;
}

__global__ void __launch_bounds__(ST)
sample_temperature_kernel(const float* __restrict__ logits, const float* __restrict__ uniforms,
                          int* __restrict__ out, int vocab, float inv_t) {
    __shared__ float red[40];
    __shared__ float warp_tot[32];
    __shared__ int chosen;
    const float* x = logits + (int64_t)blockIdx.x * vocab;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += ST) m = fmaxf(m, x[i]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    if (threadIdx.x == 0) chosen = INT_MAX;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < 32; ++w) m = fmaxf(m, red[w]);

    const int chunk = (vocab + ST - 1) / ST;
    const int lo = min(threadIdx.x * chunk, vocab), hi = min(lo + chunk, vocab);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) mine += expf((x[i] - m) * inv_t);
    float total;
    const float incl = block_scan(mine, warp_tot, &total);
    const float excl = incl - mine;
    const float target = uniforms[blockIdx.x] * total;
    if ((excl < target || threadIdx.x == 0) && incl >= target && hi > lo) {
        float run = excl;
        int pick = hi - 1;
        for (int i = lo; i < hi; ++i) {
            run += expf((x[i] - m) * inv_t);
            if (run >= target) { pick = i; break; }
        }
        atomicMin(&chosen, pick);
    }
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = chosen == INT_MAX ? vocab - 1 : chosen;
}

// Each (row, token) pair once: logit > 0 ? logit / penalty : logit * penalty
// (sampler.rs:76-85); the host removes duplicates.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, const int* __restrict__ rows,
                                          const int* __restrict__ tokens, int n, int vocab, float penalty) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = tokens[i];
    if (t < 0 || t >= vocab) return;
    float* l = logits + (int64_t)rows[i] * vocab + t;
    const float v = *l;
    *l = v > 0.f ? v / penalty : v * penalty;
}

// ---- top-k -------------------------------------------------------------------
__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);     // larger float <=> larger key (total order)
}

__global__ void __launch_bounds__(ST)
top_k_kernel(const float* __restrict__ logits, float* __restrict__ vals, int* __restrict__ idxs, int vocab, int k) {
    __shared__ unsigned hist[256];
    __shared__ unsigned long long cand[ST];
    __shared__ unsigned sh_prefix, sh_remaining, sh_count, sh_eq_taken;
    __shared__ unsigned warp_cnt[32];
    const float* x = logits + (int64_t)blockIdx.x * vocab;
    const int tid = threadIdx.x;

    // Radix select of the k-th largest key, 8 bits at a time from the top.
    if (tid == 0) { sh_prefix = 0; sh_remaining = k; }
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const unsigned prefix = sh_prefix;
        const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < vocab; i += ST) {
            const unsigned key = order_key(x[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned rem = sh_remaining;
            int bin = 255;
            for (; bin > 0; --bin) {
                if (hist[bin] >= rem) break;
                rem -= hist[bin];
            }
            sh_prefix = prefix | ((unsigned)bin << shift);
            sh_remaining = rem;
        }
        __syncthreads();
    }
    const unsigned kth = sh_prefix;            // key of the k-th largest entry
    const unsigned need_eq = sh_remaining;     // how many entries equal to it are taken (lowest indices)
    cand[tid] = 0ull;
    if (tid == 0) { sh_count = 0; sh_eq_taken = 0; }
    __syncthreads();
    for (int base = 0; base < vocab; base += ST) {
        const int i = base + tid;
        const unsigned key = i < vocab ? order_key(x[i]) : 0u;
        const bool gt = i < vocab && key > kth;
        const bool eq = i < vocab && key == kth;
        if (gt) {
            const unsigned slot = atomicAdd(&sh_count, 1u);
            cand[slot] = ((unsigned long long)key << 32) | (unsigned)(0xffffffffu - (unsigned)i);
        }
        // equal entries: taken in index order until need_eq are found
        const unsigned bal = __ballot_sync(0xffffffffu, eq);
        if ((tid & 31) == 0) warp_cnt[tid >> 5] = __popc(bal);
        __syncthreads();
        unsigned before = sh_eq_taken;
        for (int w = 0; w < (tid >> 5); ++w) before += warp_cnt[w];
        before += __popc(bal & ((1u << (tid & 31)) - 1u));
        if (eq && before < need_eq) {
            const unsigned slot = atomicAdd(&sh_count, 1u);
            cand[slot] = ((unsigned long long)key << 32) | (unsigned)(0xffffffffu - (unsigned)i);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned t = 0;
            for (int w = 0; w < 32; ++w) t += warp_cnt[w];
            sh_eq_taken += t;
        }
        __syncthreads();
    }
    // Bitonic sort, descending, of the ST slots (empty slots are zero and sink).
    for (int size = 2; size <= ST; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int partner = tid ^ stride;
            if (partner > tid) {
                const bool desc = (tid & size) == 0;
                const unsigned long long a = cand[tid], b = cand[partner];
                if ((a < b) == desc) { cand[tid] = b; cand[partner] = a; }
            }
            __syncthreads();
        }
    }
    if (tid < k) {
        const int i = (int)(0xffffffffu - (unsigned)(cand[tid] & 0xffffffffull));
        vals[(int64_t)blockIdx.x * k + tid] = x[i];
        idxs[(int64_t)blockIdx.x * k + tid] = i;
    }
}

// One token per row from k candidates sorted by logit (descending): probabilities
// exp((l - max) / T) normalised by their sum, the min-p cut, the top-p cut and one draw
// r = u * (sum of what is left) walked down the candidates (wick src/sampler.rs:95-125).
// One thread per row does the sums one after the other in float32, as the reference's
// iterator sums do (k <= 1024 on the usual path; nothing here is worth more threads).
// probs: scratch [rows, k].
__global__ void pick_sorted_kernel(const float* __restrict__ vals, const int* __restrict__ idxs, const float* __restrict__ uniforms,
                                   float* __restrict__ probs, int* __restrict__ out, int rows, int k, float temperature,
                                   float min_p, float top_p) {
    pdl_trigger();
    pdl_wait();
    vals = fresh(vals);
    idxs = fresh(idxs);
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const float* v = vals + (int64_t)row * k;
    const int* ix = idxs + (int64_t)row * k;
    float* p = probs + (int64_t)row * k;
    const float top = v[0];
    float total = 0.f;
    for (int i = 0; i < k; ++i) {
        p[i] = expf(__fdiv_rn(__fsub_rn(v[i], top), temperature));
        total = __fadd_rn(total, p[i]);
    }
    for (int i = 0; i < k; ++i) p[i] = __fdiv_rn(p[i], total);
    int keep = k;
    if (min_p > 0.f) {
        const float floor_p = __fmul_rn(p[0], min_p);
        for (int i = 0; i < k; ++i)
            if (p[i] < floor_p) { keep = i > 1 ? i : 1; break; }
    }
    if (top_p < 1.f) {
        float acc = 0.f;
        for (int i = 0; i < keep; ++i) {
            acc = __fadd_rn(acc, p[i]);
            if (acc >= top_p) { keep = i + 1; break; }
        }
    }
    float tot = 0.f;
    for (int i = 0; i < keep; ++i) tot = __fadd_rn(tot, p[i]);
    float r = __fmul_rn(uniforms[row], tot);
    int pick = ix[keep - 1];
    for (int i = 0; i < keep; ++i) {
        r = __fsub_rn(r, p[i]);
        if (r <= 0.f) { pick = ix[i]; break; }
    }
    out[row] = pick;
}

}  // namespace wick

using namespace wick;

// vals, idxs: [rows, k] candidates sorted by value (descending); uniforms: [rows] in [0, 1);
// probs: float32 scratch [rows, k]; out: int32 [rows].
WICK_API int wick_pick_sorted(const float* vals, const int* idxs, const float* uniforms, float* probs, int* out, int rows, int k,
                              float temperature, float min_p, float top_p, void* s) {
    WICK_REQUIRE(rows >= 0 && k >= 1 && temperature > 0.f, "pick_sorted: bad arguments");
    if (rows == 0) return 0;
    WICK_CUDA(launch(pick_sorted_kernel, dim3(ceil_div(rows, 32)), dim3(32), 0, (cudaStream_t)s, vals, idxs, uniforms, probs, out,
                     rows, k, temperature, min_p, top_p));
    return check_launch("pick_sorted");
}

WICK_API int wick_argmax(const float* logits, int* out, int rows, int vocab, void* s) {
    WICK_REQUIRE(vocab > 0 && rows >= 0, "argmax: bad sizes");
    if (rows == 0) return 0;
    WICK_CUDA(launch(argmax_kernel, dim3(rows), dim3(ST), 0, (cudaStream_t)s, logits, out, vocab));
    return check_launch("argmax");
}

WICK_API int wick_sample_temperature(const float* logits, const float* uniforms, int* out, int rows, int vocab,
                                     float inv_t, void* s) {
    WICK_REQUIRE(vocab > 0 && rows >= 0 && inv_t > 0.f, "sample_temperature: bad arguments");
    if (rows == 0) return 0;
    sample_temperature_kernel<<<rows, ST, 0, (cudaStream_t)s>>>(logits, uniforms, out, vocab, inv_t);
    return check_launch("sample_temperature");
}

WICK_API int wick_top_k(const float* logits, float* vals, int* idxs, int rows, int vocab, int k, void* s) {
    WICK_REQUIRE(vocab > 0 && rows >= 0, "top_k: bad sizes");
    WICK_REQUIRE(k >= 1 && k <= ST && k <= vocab, "top_k: k=%d must lie in [1, min(vocab, %d)]", k, ST);
    if (rows == 0) return 0;
    top_k_kernel<<<rows, ST, 0, (cudaStream_t)s>>>(logits, vals, idxs, vocab, k);
    return check_launch("top_k");
}

WICK_API int wick_repetition_penalty(float* logits, const int* rows, const int* tokens, int n, int vocab,
                                     float penalty, void* s) {
    WICK_REQUIRE(vocab > 0 && n >= 0, "repetition_penalty: bad sizes");
    if (n == 0) return 0;
    repetition_penalty_kernel<<<ceil_div(n, 256), 256, 0, (cudaStream_t)s>>>(logits, rows, tokens, n, vocab, penalty);
    return check_launch("repetition_penalty");
}
