// Row-wise kernels of the decoder: embedding gather, RMSNorm (optionally fused
// with the residual addition and with a row gather), rotary tables, the fused
// per-head norm + rotation + cache append, and SwiGLU on separate arrays.
//
// All arithmetic is float32; T is the storage type of activations (bfloat16 or
// float).  Formulas: wick src/kernels.rs:343-357 (rms norm: sum of squares over
// the row, divided by its length, scale = 1/sqrt(ss+eps), (x*scale)*w),
// src/model.rs:404-414 (half-split rotation by pos*inv_freq[i]),
// src/model.rs:475-483 (norm, then rotation, then the cache write),
// src/kernels.rs:374-378 (g/(1+exp(-g))*u).
#include "common.cuh"

namespace wick {


// Eight neighbouring elements at a 16-byte aligned place, as float32.
__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        v[2 * k] = f.x;
        v[2 * k + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

// ---- embedding -------------------------------------------------------------
// vec: the width is a multiple of 8 and the table is 16-byte aligned (eight elements a load).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int width, int vec) {
    pdl_trigger();
    pdl_wait();
    const int64_t row = blockIdx.x;
    const T* src = table + (int64_t)tokens[row] * width;
    float* dst = out + row * width;
    if (vec) {
        for (int j = threadIdx.x * 8; j < width; j += blockDim.x * 8) {
            float v[8];
            load8(src + j, v);
            store8(dst + j, v);
        }
        return;
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = ld(src + j);
}

// ---- RMSNorm ---------------------------------------------------------------
// Two kernels compute it: one block per row (few rows: a decode step) and one warp
// per row (many rows: a prompt).  They give the same bits.  The sum of squares of a row
// whose width is a multiple of 4 is defined as: every four neighbouring elements' own sum
// (sumsq4 from zero); those, 32 apart, added up in index order (class c: quads c, c + 32,
// ...); the 32 class sums by the butterfly.  A lane of the warp kernel holds exactly one
// class; the block kernel leaves the quads' sums in shared memory and its first warp adds
// up the classes.  The operations are spelled out so that the compiler contracts nothing
// differently in the two.
__device__ __forceinline__ float sumsq4(float ss, float4 v) {
    return __fadd_rn(ss, __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(v.x, v.x), __fmul_rn(v.y, v.y)), __fmul_rn(v.z, v.z)), __fmul_rn(v.w, v.w)));
}
__device__ __forceinline__ float normed(float v, float scale, float g) { return __fmul_rn(__fmul_rn(v, scale), g); }
// Four neighbouring outputs at an index that is a multiple of 4.
__device__ __forceinline__ void st4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float a, float b, float c, float d) {
    uint2 u;
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float rms_scale(float ss, int width, float eps) { return 1.0f / sqrtf(__fadd_rn(__fdiv_rn(ss, (float)width), eps)); }

// One block per output row i.  Source row r = rows ? rows[i] : i.  If delta is
// given, x[r] + delta[0][r] + delta[1][r] + ... (index order) is normalised; without
// `rows` the sum is also written back to x.  With `rows` x stays as it is: a row may be
// named twice, and two blocks that both wrote it back could each read the other's sum.
template <typename TOut>
__global__ void __launch_bounds__(1024, 1) rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits,
                               int64_t split_stride, const float* __restrict__ w, float eps,
                               const int* __restrict__ rows, TOut* __restrict__ out, int width) {
    extern __shared__ float smem[];
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    delta = fresh(delta);
    float* row = smem;
    float* red = smem + width;
    float* quads = red + 40;                            // [width / 4] sums of four neighbouring squares
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* xr = x + r * width;
    float ss = 0.f;
    if ((width & 3) == 0) {
        // four floats per thread and iteration; all loads of an iteration are independent
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(xr + j);
            if (delta) {
                for (int s = 0; s < splits; ++s) {
                    const float4 d = *reinterpret_cast<const float4*>(delta + s * split_stride + r * width + j);
                    v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                }
                if (!rows) *reinterpret_cast<float4*>(xr + j) = v;      // (selected rows: x stays, see below)
            }
            *reinterpret_cast<float4*>(row + j) = v;
            quads[j >> 2] = sumsq4(0.f, v);
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            float p = 0.f;
            for (int q = threadIdx.x; q < (width >> 2); q += 32) p = __fadd_rn(p, quads[q]);
            p = warp_sum(p);
            if (threadIdx.x == 0) red[0] = p;
        }
        __syncthreads();
        ss = red[0];
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            float v = xr[j];
            if (delta) {
                for (int s = 0; s < splits; ++s) v += delta[s * split_stride + r * width + j];
                if (!rows) xr[j] = v;
            }
            row[j] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
    }
    const float scale = rms_scale(ss, width, eps);
    TOut* o = out + (int64_t)i * width;
    if ((width & 3) == 0) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + j);
            const float4 g = *reinterpret_cast<const float4*>(w + j);
            st(o + j, normed(v.x, scale, g.x));
            st(o + j + 1, normed(v.y, scale, g.y));
            st(o + j + 2, normed(v.z, scale, g.z));
            st(o + j + 3, normed(v.w, scale, g.w));
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) st(o + j, (row[j] * scale) * w[j]);
    }
}

// One warp per output row, for rows that are a multiple of 4 wide and at most 4096:
// the row stays in registers (lane l holds quads l, l + 32, ...: one class of the sum),
// nothing is synchronised but the warp.
template <typename TOut>
__global__ void __launch_bounds__(128) rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits,
                                                           int64_t split_stride, const float* __restrict__ w, float eps,
                                                           const int* __restrict__ rows, TOut* __restrict__ out, int n_out,
                                                           int width) {
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    delta = fresh(delta);
    constexpr int QMAX = 4096 / 4 / 32;                 // quads of a lane
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= n_out) return;
    const int64_t r = rows ? rows[i] : i;
    float* xr = x + r * width;
    float4 v[QMAX];
#pragma unroll
    for (int m = 0; m < QMAX; ++m) {
        const int j = (lane + 32 * m) * 4;
        v[m] = j < width ? *reinterpret_cast<const float4*>(xr + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (delta) {
        for (int s = 0; s < splits; ++s) {
#pragma unroll
            for (int m = 0; m < QMAX; ++m) {
                const int j = (lane + 32 * m) * 4;
                if (j < width) {
                    const float4 d = *reinterpret_cast<const float4*>(delta + s * split_stride + r * width + j);
                    v[m].x += d.x; v[m].y += d.y; v[m].z += d.z; v[m].w += d.w;
                }
            }
        }
#pragma unroll
        for (int m = 0; m < QMAX; ++m) {
            const int j = (lane + 32 * m) * 4;
            if (j < width && !rows) *reinterpret_cast<float4*>(xr + j) = v[m];
        }
    }
    float p = 0.f;
#pragma unroll
    for (int m = 0; m < QMAX; ++m)
        if ((lane + 32 * m) * 4 < width) p = __fadd_rn(p, sumsq4(0.f, v[m]));
    const float scale = rms_scale(warp_sum(p), width, eps);
    TOut* o = out + (int64_t)i * width;
#pragma unroll
    for (int m = 0; m < QMAX; ++m) {
        const int j = (lane + 32 * m) * 4;
        if (j < width) {
            const float4 g = *reinterpret_cast<const float4*>(w + j);
            const float4 q = v[m];
            st4(o + j, normed(q.x, scale, g.x), normed(q.y, scale, g.y), normed(q.z, scale, g.z), normed(q.w, scale, g.w));
        }
    }
}

// x[r] += sum of delta for every row (no norm): resolves a pending residual.
__global__ void add_delta_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits,
                                 int64_t split_stride, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    for (int s = 0; s < splits; ++s) v += delta[s * split_stride + i];
    x[i] = v;
}

// ---- rotary tables ---------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t, int n, int half) {
    pdl_trigger();
    pdl_wait();
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)n * half) return;
    const int t = idx / half, i = idx % half;
    const float angle = (float)positions[t] * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    cos_t[idx] = c;
    sin_t[idx] = s;
}

// Two neighbouring elements at an even index.
__device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void st2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void st2(__nv_bfloat16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }

// ---- per-head norm + rotation + cache append --------------------------------
// One warp per (token, head) vector of the fused projection output
// qkv[token] = [q heads | k heads | v heads].  q goes to q_out, k and v go to the
// token's place in its sequence's cache page.  A warp takes HB vectors in a row and
// issues the loads of all of them before it uses the first (a prompt's kernel is
// bound by how many loads are in flight, not by arithmetic).
template <typename T, int HB>
__global__ void qk_norm_rope_append_kernel(
    const T* __restrict__ qkv, const float* __restrict__ parts, int splits, int64_t split_stride,
    int n_tokens, int n_heads, int n_kv, int hd,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    T* __restrict__ q_out, T* __restrict__ kv, const int* __restrict__ page_table, int table_width,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions, int write_kv) {
    pdl_trigger();
    pdl_wait();
    qkv = fresh(qkv);
    parts = fresh(parts);
    cos_t = fresh(cos_t);
    sin_t = fresh(sin_t);
    const int lane = threadIdx.x & 31;
    const int heads_total = n_heads + (write_kv ? 2 * n_kv : 0);
    // grid: (tokens, groups of heads): no division to find a vector's token and head
    const int t = blockIdx.x;
    const int h0 = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * HB;
    if (h0 >= heads_total) return;
    const int half = hd >> 1;
    const int row_width = (n_heads + 2 * n_kv) * hd;
    // A lane holds, for i = 2 lane (+ 64, ...) below head_dim / 2, the elements i, i + 1 and
    // their partners in the rotation, i + head_dim / 2 and i + 1 + head_dim / 2: everything
    // it needs is loaded once.  head_dim <= 256: at most two such groups.
    constexpr int MAXG = 2;
    float2 xa[HB][MAXG], xb[HB][MAXG];
#pragma unroll
    for (int u = 0; u < HB; ++u) {
        const int h = h0 + u;
        if (h >= heads_total) break;
        // The projection output comes either as one array of T or as float32 partial
        // sums [splits][tokens][row_width] that are added here, in index order.
        const int64_t base = (int64_t)t * row_width + (int64_t)h * hd;
        auto val2 = [&](int i) -> float2 {
            if (parts) {
                float2 v = *reinterpret_cast<const float2*>(parts + base + i);
                for (int sp = 1; sp < splits; ++sp) {
                    const float2 d = *reinterpret_cast<const float2*>(parts + sp * split_stride + base + i);
                    v.x += d.x;
                    v.y += d.y;
                }
                return v;
            }
            return ld2(qkv + base + i);
        };
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
            const int i = 2 * lane + 64 * g;
            if (i < half) {
                xa[u][g] = val2(i);
                xb[u][g] = val2(i + half);
            }
        }
    }
    // The token's angles and both norm weights are asked for now, with the vectors: one
    // trip to the memory instead of three in a row.
    float2 cs[MAXG], sn[MAXG], wq[MAXG][2], wk[MAXG][2];
    const bool has_k = write_kv && h0 + HB > n_heads;
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
        const int i = 2 * lane + 64 * g;
        cs[g] = sn[g] = wq[g][0] = wq[g][1] = wk[g][0] = wk[g][1] = make_float2(0.f, 0.f);
        if (i < half) {
            if (cos_t) {
                cs[g] = *reinterpret_cast<const float2*>(cos_t + (int64_t)t * half + i);
                sn[g] = *reinterpret_cast<const float2*>(sin_t + (int64_t)t * half + i);
            }
            if (q_w && h0 < n_heads) {
                wq[g][0] = *reinterpret_cast<const float2*>(q_w + i);
                wq[g][1] = *reinterpret_cast<const float2*>(q_w + i + half);
            }
            if (k_w && has_k) {
                wk[g][0] = *reinterpret_cast<const float2*>(k_w + i);
                wk[g][1] = *reinterpret_cast<const float2*>(k_w + i + half);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < HB; ++u) {
        const int h = h0 + u;
        if (h >= heads_total) break;
        T* dst;
        const float* w = nullptr;
        bool rotate = true;
        if (h < n_heads) {
            dst = q_out + ((int64_t)t * n_heads + h) * hd;
            w = q_w;
        } else {
            const int is_v = h >= n_heads + n_kv;
            const int kh = h - n_heads - (is_v ? n_kv : 0);
            const int pos = positions[t];
            const int page = page_table[(int64_t)seq_of_token[t] * table_width + pos / kPage];
            dst = kv + ((((int64_t)page * 2 + is_v) * n_kv + kh) * kPage + (pos % kPage)) * hd;
            w = is_v ? nullptr : k_w;
            rotate = !is_v;                                    // the value goes into the cache as it is
        }
        float scale = 1.f;
        if (w) {
            float ss = 0.f;
#pragma unroll
            for (int g = 0; g < MAXG; ++g)
                if (2 * lane + 64 * g < half)
                    ss += xa[u][g].x * xa[u][g].x + xa[u][g].y * xa[u][g].y + xb[u][g].x * xb[u][g].x + xb[u][g].y * xb[u][g].y;
            ss = warp_sum(ss);
            scale = 1.0f / sqrtf(ss / (float)hd + eps);
        }
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
            const int i = 2 * lane + 64 * g;
            if (i < half) {
                float2 a = xa[u][g], b = xb[u][g];
                if (w) {
                    const float2 wa = h < n_heads ? wq[g][0] : wk[g][0], wb = h < n_heads ? wq[g][1] : wk[g][1];
                    a.x = (a.x * scale) * wa.x;
                    a.y = (a.y * scale) * wa.y;
                    b.x = (b.x * scale) * wb.x;
                    b.y = (b.y * scale) * wb.y;
                }
                if (rotate && cos_t) {
                    const float2 c = cs[g], s2 = sn[g];
                    const float rax = a.x * c.x - b.x * s2.x, rbx = b.x * c.x + a.x * s2.x;
                    const float ray = a.y * c.y - b.y * s2.y, rby = b.y * c.y + a.y * s2.y;
                    a = make_float2(rax, ray);
                    b = make_float2(rbx, rby);
                }
                st2(dst + i, a);
                st2(dst + i + half, b);
            }
        }
    }
}

// The same for head sizes in steps of 16 with 16-byte aligned arrays: L lanes per vector
// (L * 8 >= head_dim / 2; a lane holds 8 neighbouring elements and their 8 partners in
// the rotation), so that a warp takes 32 / L vectors with one stream of instructions.
// The first form spends ~240 instructions per vector and is bound by their issue (the
// square root and the divisions of the scale above all, once per vector whatever the
// number of lanes); this one issues them once per 32 / L vectors.
template <typename T, int L>
__global__ void __launch_bounds__(128)
qk_norm_rope_append_vec_kernel(
    const T* __restrict__ qkv, const float* __restrict__ parts, int splits, int64_t split_stride,
    int n_tokens, int n_heads, int n_kv, int hd,
    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    T* __restrict__ q_out, T* __restrict__ kv, const int* __restrict__ page_table, int table_width,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions, int write_kv) {
    pdl_trigger();
    pdl_wait();
    qkv = fresh(qkv);
    parts = fresh(parts);
    cos_t = fresh(cos_t);
    sin_t = fresh(sin_t);
    const int heads_total = n_heads + (write_kv ? 2 * n_kv : 0);
    const int t = blockIdx.x;
    const int h = (blockIdx.y * blockDim.x + threadIdx.x) / L;      // this group of lanes' vector
    const int half = hd >> 1;
    const int i0 = (threadIdx.x % L) * 8;                           // the lane's elements i0 .. i0 + 7 and i0 + half ..
    const bool live = h < heads_total && i0 < half;                 // (every lane stays for the shuffles)
    const int row_width = (n_heads + 2 * n_kv) * hd;
    float a[8], b[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = b[k] = 0.f;
    float c[8], sn[8], wa[8], wb[8];
    const bool is_q = h < n_heads, is_v = h >= n_heads + n_kv;
    const float* w = is_q ? q_w : (is_v ? nullptr : k_w);
    const bool rotate = !is_v && cos_t != nullptr;
    T* dst = nullptr;
    if (live) {
        const int64_t base = (int64_t)t * row_width + (int64_t)h * hd + i0;
        if (parts) {
            // float32 partial sums [splits][tokens][row_width], added in index order
            load8(parts + base, a);
            load8(parts + base + half, b);
            for (int sp = 1; sp < splits; ++sp) {
                float da[8], db[8];
                load8(parts + sp * split_stride + base, da);
                load8(parts + sp * split_stride + base + half, db);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    a[k] += da[k];
                    b[k] += db[k];
                }
            }
        } else {
            load8(qkv + base, a);
            load8(qkv + base + half, b);
        }
        if (rotate) {
            load8(cos_t + (int64_t)t * half + i0, c);
            load8(sin_t + (int64_t)t * half + i0, sn);
        }
        if (w) {
            load8(w + i0, wa);
            load8(w + i0 + half, wb);
        }
        if (is_q) dst = q_out + ((int64_t)t * n_heads + h) * hd + i0;
        else {
            const int kh = h - n_heads - (is_v ? n_kv : 0);
            const int pos = positions[t];
            const int page = page_table[(int64_t)seq_of_token[t] * table_width + pos / kPage];
            dst = kv + ((((int64_t)page * 2 + (is_v ? 1 : 0)) * n_kv + kh) * kPage + (pos % kPage)) * hd + i0;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += a[k] * a[k] + b[k] * b[k];
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!live) return;
    if (w) {
        const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            a[k] = (a[k] * scale) * wa[k];
            b[k] = (b[k] * scale) * wb[k];
        }
    }
    if (rotate) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float ra = a[k] * c[k] - b[k] * sn[k], rb = b[k] * c[k] + a[k] * sn[k];
            a[k] = ra;
            b[k] = rb;
        }
    }
    store8(dst, a);
    store8(dst + half, b);
}

// ---- SwiGLU on separate arrays ----------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                                int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = ld(gate + i), u = ld(up + i);
    st(out + i, g / (1.0f + expf(-g)) * u);
}

template <typename T>
int embed(const void* table, const int* tokens, float* out, int n, int width, int64_t vocab, cudaStream_t s) {
    WICK_REQUIRE(n >= 0 && width > 0 && vocab > 0, "embed: bad sizes n=%d width=%d", n, width);
    if (n == 0) return 0;
    const int vec = width % 8 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0;
    WICK_CUDA(launch(embed_kernel<T>, dim3(n), dim3(256), 0, s, (const T*)table, tokens, out, width, vec));
    return check_launch("embed");
}

template <typename TOut>
int rmsnorm(float* x, const float* delta, int splits, int64_t n_rows_x, const float* w, float eps,
            const int* rows, void* out, int n_out, int width, cudaStream_t s) {
    WICK_REQUIRE(width > 0 && n_out >= 0, "rmsnorm: bad sizes");
    if (n_out == 0) return 0;
    const size_t smem = ((size_t)width + 40 + width / 4 + 1) * sizeof(float);
    WICK_REQUIRE(smem <= 200 * 1024, "rmsnorm: width %d is beyond the %d that one block's shared memory holds",
                 width, (200 * 1024 / 4 - 41) * 4 / 5);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        WICK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    const int threads = width >= 4096 ? 1024 : (width >= 2048 ? 512 : (width >= 512 ? 256 : 128));
    if (n_out >= 512 && width % 4 == 0 && width <= 4096) {
        // Enough rows to give every SM its warps: a warp per row (same bits as the block per row).
        // With fewer rows (a decode step of 64 sequences) a warp per row leaves most of the part
        // idle and each warp walks its row's partial sums alone: the block per row is 3x faster there.
        const dim3 grid(ceil_div(n_out, 4)), block(128);
        const int64_t stride = n_rows_x * width;
        WICK_CUDA(launch(rmsnorm_rows_kernel<TOut>, grid, block, 0, s, x, delta, splits, stride, w, eps, rows, (TOut*)out, n_out, width));
        return check_launch("rmsnorm");
    }
    WICK_CUDA(launch(rmsnorm_kernel<TOut>, dim3(n_out), dim3(threads), smem, s, x, delta, splits, n_rows_x * width, w,
                     eps, rows, (TOut*)out, width));
    return check_launch("rmsnorm");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;


WICK_API int wick_embed_bf16(const void* table, const int* tokens, float* out, int n, int width, int64_t vocab, void* s) {
    return embed<bf16>(table, tokens, out, n, width, vocab, (cudaStream_t)s);
}
WICK_API int wick_embed_f32(const void* table, const int* tokens, float* out, int n, int width, int64_t vocab, void* s) {
    return embed<float>(table, tokens, out, n, width, vocab, (cudaStream_t)s);
}

// x: float32 [n_rows_x, width] (updated in place when delta is given);
// delta: float32 [splits, n_rows_x, width] or null; rows: int32 [n_out] or null
// (then n_out == n_rows_x); out: [n_out, width].
WICK_API int wick_rmsnorm_bf16(float* x, const float* delta, int splits, int64_t n_rows_x, const float* w, float eps,
                               const int* rows, void* out, int n_out, int width, void* s) {
    return rmsnorm<bf16>(x, delta, splits, n_rows_x, w, eps, rows, out, n_out, width, (cudaStream_t)s);
}
WICK_API int wick_rmsnorm_f32(float* x, const float* delta, int splits, int64_t n_rows_x, const float* w, float eps,
                              const int* rows, void* out, int n_out, int width, void* s) {
    return rmsnorm<float>(x, delta, splits, n_rows_x, w, eps, rows, out, n_out, width, (cudaStream_t)s);
}

WICK_API int wick_add_delta(float* x, const float* delta, int splits, int64_t n, void* s) {
    if (n == 0) return 0;
    add_delta_kernel<<<ceil_div(n, 256), 256, 0, (cudaStream_t)s>>>(x, delta, splits, n, n);
    return check_launch("add_delta");
}

WICK_API int wick_rope_table(const int* positions, const float* inv_freq, float* cos_t, float* sin_t, int n,
                             int half, void* s) {
    if (n == 0 || half == 0) return 0;
    WICK_CUDA(launch(rope_table_kernel, dim3(ceil_div((int64_t)n * half, 256)), dim3(256), 0, (cudaStream_t)s, positions,
                     inv_freq, cos_t, sin_t, n, half));
    return check_launch("rope_table");
}

template <typename T>
static int qk_norm_rope_append(const void* qkv, const float* parts, int splits, int n_tokens, int n_heads, int n_kv, int hd, const float* q_w,
                               const float* k_w, float eps, const float* cos_t, const float* sin_t, void* q_out,
                               void* kv, const int* page_table, int table_width, const int* seq_of_token,
                               const int* positions, int write_kv, cudaStream_t s) {
    WICK_REQUIRE(hd > 0 && hd % 4 == 0 && hd <= 256, "qk_norm_rope_append: head_dim %d must be a multiple of 4 up to 256", hd);
    WICK_REQUIRE(n_heads > 0 && n_kv > 0, "qk_norm_rope_append: bad head counts");
    if (n_tokens == 0) return 0;
    const int heads_total = n_heads + (write_kv ? 2 * n_kv : 0);
    const int warps = 4;
    const int64_t stride = (int64_t)n_tokens * (n_heads + 2 * n_kv) * hd;
    WICK_REQUIRE(heads_total <= 65535 * warps, "qk_norm_rope_append: %d heads is beyond the grid limit", heads_total);
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (hd % 16 == 0 && (stride * (int64_t)sizeof(float)) % 16 == 0 && aligned(qkv) && aligned(parts) && aligned(q_w) && aligned(k_w) &&
        aligned(cos_t) && aligned(sin_t) && aligned(q_out) && aligned(kv)) {
        // L lanes of 8 elements (and their partners) per vector
        const int lanes = hd <= 64 ? 4 : (hd <= 128 ? 8 : 16);
        const dim3 grid(n_tokens, ceil_div((int64_t)heads_total * lanes, warps * 32)), block(warps * 32);
#define WICK_QK_VEC(L)                                                                                                         \
    WICK_CUDA(launch(qk_norm_rope_append_vec_kernel<T, L>, grid, block, 0, s, (const T*)qkv, parts, splits, stride, n_tokens, n_heads, \
                     n_kv, hd, q_w, k_w, eps, cos_t, sin_t, (T*)q_out, (T*)kv, page_table, table_width, seq_of_token, positions, write_kv))
        if (lanes == 4) WICK_QK_VEC(4);
        else if (lanes == 8) WICK_QK_VEC(8);
        else WICK_QK_VEC(16);
#undef WICK_QK_VEC
        return check_launch("qk_norm_rope_append");
    }
    if ((int64_t)n_tokens * heads_total >= 8192) {            // a prompt: two vectors per warp
        WICK_CUDA(launch(qk_norm_rope_append_kernel<T, 2>, dim3(n_tokens, ceil_div(heads_total, warps * 2)), dim3(warps * 32), 0, s,
                         (const T*)qkv, parts, splits, stride, n_tokens, n_heads, n_kv, hd, q_w, k_w, eps, cos_t, sin_t, (T*)q_out,
                         (T*)kv, page_table, table_width, seq_of_token, positions, write_kv));
    } else {
        WICK_CUDA(launch(qk_norm_rope_append_kernel<T, 1>, dim3(n_tokens, ceil_div(heads_total, warps)), dim3(warps * 32), 0, s,
                         (const T*)qkv, parts, splits, stride, n_tokens, n_heads, n_kv, hd, q_w, k_w, eps, cos_t, sin_t, (T*)q_out,
                         (T*)kv, page_table, table_width, seq_of_token, positions, write_kv));
    }
    return check_launch("qk_norm_rope_append");
}

WICK_API int wick_qk_norm_rope_append_bf16(const void* qkv, const float* parts, int splits, int n_tokens, int n_heads, int n_kv, int hd,
                                           const float* q_w, const float* k_w, float eps, const float* cos_t,
                                           const float* sin_t, void* q_out, void* kv, const int* page_table,
                                           int table_width, const int* seq_of_token, const int* positions,
                                           int write_kv, void* s) {
    return qk_norm_rope_append<bf16>(qkv, parts, splits, n_tokens, n_heads, n_kv, hd, q_w, k_w, eps, cos_t, sin_t, q_out, kv,
                                     page_table, table_width, seq_of_token, positions, write_kv, (cudaStream_t)s);
}
WICK_API int wick_qk_norm_rope_append_f32(const void* qkv, const float* parts, int splits, int n_tokens, int n_heads, int n_kv, int hd,
                                          const float* q_w, const float* k_w, float eps, const float* cos_t,
                                          const float* sin_t, void* q_out, void* kv, const int* page_table,
                                          int table_width, const int* seq_of_token, const int* positions,
                                          int write_kv, void* s) {
    return qk_norm_rope_append<float>(qkv, parts, splits, n_tokens, n_heads, n_kv, hd, q_w, k_w, eps, cos_t, sin_t, q_out, kv,
                                      page_table, table_width, seq_of_token, positions, write_kv, (cudaStream_t)s);
}

WICK_API int wick_silu_mul_bf16(const void* g, const void* u, void* out, int64_t n, void* s) {
    if (n == 0) return 0;
    silu_mul_kernel<bf16><<<ceil_div(n, 256), 256, 0, (cudaStream_t)s>>>((const bf16*)g, (const bf16*)u, (bf16*)out, n);
    return check_launch("silu_mul");
}
WICK_API int wick_silu_mul_f32(const void* g, const void* u, void* out, int64_t n, void* s) {
    if (n == 0) return 0;
    silu_mul_kernel<float><<<ceil_div(n, 256), 256, 0, (cudaStream_t)s>>>((const float*)g, (const float*)u, (float*)out, n);
    return check_launch("silu_mul");
}
