// Row-wise kernels: embedding, residual add + RMSNorm, q/k head norm + RoPE + cache write,
// SwiGLU.  Each is templated on the activation type (float for the 32-bit path, bfloat16 for
// the serving path); per-channel weights are always float32.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512];

void x0ne_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

X0NE_API const char* x0ne_last_error() { return g_error; }

bool x0ne_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("X0NE_PDL");
        on = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}


// ----------------------------------------------------------------------------------------
// Residual add, then RMSNorm: r = resid + f32(delta) (one IEEE add, stored back);
// out = T(r * rsqrt(mean(r^2) + eps) * w)  (x0ne-core/kernels/cuda/rmsnorm.cu:11-20; eps is
// inside the root; the weight multiplies directly).  `delta` may be null (norm only).
// `rows`, if given, lists the source rows to process; output row i then belongs to source row
// rows[i] (used to norm only the rows whose logits are wanted).
// One block per row; the sum of squares is a fixed-order block sum.
// ----------------------------------------------------------------------------------------
// General form, any width: each thread owns every blockDim-th element.  The row after the add is
// parked in shared memory between the two sweeps when it fits there (`keep` floats of dynamic
// shared memory, 0 if it does not), so the residual is read once.
template <typename T>
__global__ void add_rmsnorm_any_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ out,
                                       const int32_t* __restrict__ rows, int hidden, float eps, int keep) {
    extern __shared__ float parked[];
    __shared__ float partial[32];
    pdl_prologue();
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = resid + src * hidden;
    float sum_sq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = r[i];
        if (delta) {
            v = v + to_f32(delta[src * hidden + i]);     // one IEEE add, stored back
            r[i] = v;
        }
        if (i < keep) parked[i] = v;
        sum_sq = fmaf(v, v, sum_sq);
    }
    const float mean_sq = block_reduce(sum_sq, partial, OpSum(), 0.f) / (float)hidden;
    const float scale = 1.0f / sqrtf(mean_sq + eps);
    T* o = out + (int64_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = i < keep ? parked[i] : r[i];     // a thread reads back only what it wrote itself
        o[i] = from_f32<T>(v * scale * w[i]);
    }
}

// The same, for hidden % 8 == 0 and hidden <= 8 * 1024 * VEC_IT: 16-byte accesses, and the row stays
// in registers between the sum of squares and the scaling, so it is read once.
#define VEC_IT 4
__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float* v) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ void load2(const float* p, float* v) {
    const float2 a = *reinterpret_cast<const float2*>(p);
    v[0] = a.x; v[1] = a.y;
}
__device__ __forceinline__ void load2(const bf16* p, float* v) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    v[0] = f.x; v[1] = f.y;
}
__device__ __forceinline__ void store2(float* p, const float* v) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
__device__ __forceinline__ void store2(bf16* p, const float* v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
}
__device__ __forceinline__ void copy16(float* d, const float* s) {    // 8 values
    reinterpret_cast<float4*>(d)[0] = reinterpret_cast<const float4*>(s)[0];
    reinterpret_cast<float4*>(d)[1] = reinterpret_cast<const float4*>(s)[1];
}
__device__ __forceinline__ void copy16(bf16* d, const bf16* s) { *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s); }
__device__ __forceinline__ void copy2(float* d, const float* s) { *reinterpret_cast<float2*>(d) = *reinterpret_cast<const float2*>(s); }
__device__ __forceinline__ void copy2(bf16* d, const bf16* s) { *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(s); }

// ITS: how many sweeps of the block cover a row (1, 2 or VEC_IT).
template <typename T, int ITS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ out,
                                       const int32_t* __restrict__ rows, int hidden, float eps) {
    __shared__ float sh[32];
    // The weight and the list of rows are older than any kernel still running: they are asked for
    // before the wait for the kernel before this one, so that its end is followed by one trip to
    // memory (the row) and not by two.  (With four sweeps the weight would not fit in the registers
    // that 1,024 threads can have; it is read after the sum then.)
    constexpr bool EARLY = ITS <= 2;
    pdl_launch_dependents();
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float wv[EARLY ? ITS : 1][8];
    if (EARLY) {
#pragma unroll
        for (int it = 0; it < ITS; ++it) {
            const int i = (it * blockDim.x + threadIdx.x) * 8;
            if (i < hidden) load8(w + i, wv[it]);
        }
    }
    pdl_wait();
    float* r = resid + src * hidden;
    const T* d = delta ? delta + src * hidden : nullptr;
    T* o = out + (int64_t)blockIdx.x * hidden;
    float v[ITS][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITS; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 8;
        if (i < hidden) {
            load8(r + i, v[it]);
            if (d) {
                float dv[8];
                load8(d + i, dv);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[it][k] = v[it][k] + dv[k];
                store8(r + i, v[it]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += v[it][k] * v[it][k];
        }
    }
    const float total = block_sum(ss, sh);
    const float scale = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < ITS; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 8;
        if (i < hidden) {
            float late[8], ov[8];
            if (!EARLY) load8(w + i, late);
#pragma unroll
            for (int k = 0; k < 8; ++k) ov[k] = v[it][k] * scale * (EARLY ? wv[EARLY ? it : 0][k] : late[k]);
            store8(o + i, ov);
        }
    }
}

template <typename T>
static void launch_add_rmsnorm_vec(float* resid, const T* delta, const float* w, T* out, const int32_t* rows, int n_rows,
                                   int hidden, float eps, int threads, cudaStream_t stream) {
    const int sweeps = (hidden / 8 + threads - 1) / threads;
    if (sweeps <= 1)
        x0ne_launch(add_rmsnorm_vec_kernel<T, 1>, dim3(n_rows), dim3(threads), 0, stream, resid, delta, w, out, rows, hidden, eps);
    else if (sweeps == 2)
        x0ne_launch(add_rmsnorm_vec_kernel<T, 2>, dim3(n_rows), dim3(threads), 0, stream, resid, delta, w, out, rows, hidden, eps);
    else
        x0ne_launch(add_rmsnorm_vec_kernel<T, VEC_IT>, dim3(n_rows), dim3(threads), 0, stream, resid, delta, w, out, rows, hidden, eps);
}

X0NE_API int x0ne_add_rmsnorm(float* resid, const void* delta, const float* w, void* out, int dt,
                              const int32_t* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: rows %d hidden %d", n_rows, hidden);
    if (n_rows == 0) return 0;
    if (hidden % 8 == 0 && hidden <= 8 * 1024 * VEC_IT &&
        ((((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) == 0)) {
        int threads = (hidden / 8 + 31) / 32 * 32;
        if (threads > 1024) threads = 1024;
        if (hidden / 8 > 512 && hidden / 8 <= 1024) threads = 512;   // two sweeps of 512 rather than one of 1024
        if (dt == X0NE_F32)
            launch_add_rmsnorm_vec<float>(resid, (const float*)delta, w, (float*)out, rows, n_rows, hidden, eps, threads, stream);
        else if (dt == X0NE_BF16)
            launch_add_rmsnorm_vec<bf16>(resid, (const bf16*)delta, w, (bf16*)out, rows, n_rows, hidden, eps, threads, stream);
        else
            X0NE_REQUIRE(false, "add_rmsnorm: unknown dtype tag %d", dt);
        X0NE_LAUNCH_CHECK();
    }
    const int block = 256;
    const int keep = hidden <= 10240 ? hidden : 0;        // up to 40 KB of dynamic shared memory
    const size_t smem = (size_t)keep * sizeof(float);
    if (dt == X0NE_F32)
        x0ne_launch(add_rmsnorm_any_kernel<float>, dim3(n_rows), dim3(block), smem, stream, resid, (const float*)delta, w, (float*)out, rows, hidden, eps, keep);
    else if (dt == X0NE_BF16)
        x0ne_launch(add_rmsnorm_any_kernel<bf16>, dim3(n_rows), dim3(block), smem, stream, resid, (const bf16*)delta, w, (bf16*)out, rows, hidden, eps, keep);
    else
        X0NE_REQUIRE(false, "add_rmsnorm: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Per-head RMSNorm of q and k (optional), rotate-half RoPE, and the K/V write into the
// paged cache (x0ne-core/kernels/cuda/rope.cu:7-47).  One warp per (row, head); the row's sines and
// cosines come from a table made at start-up (or are computed by the warp); heads
// 0..q_heads-1 are q heads, the rest k heads, whose warps also copy the v head.
//   scale = rsqrt(mean(x^2 over head_dim) + eps); n = x * scale * w
//   angle = (float)pos * inv_freq[i]; (a, b) = (n[i], n[i + rot/2])
//   out[i] = a cos - b sin; out[i + rot/2] = b cos + a sin; dims >= rot pass through.
// `norm_q`/`norm_k` null: no head norm.  rot == 0: no rotation.
// A row whose position has no page writes nothing into the cache.
// ----------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void rope_one_head(const T* __restrict__ qkv, const float* __restrict__ norm_q,
                                              const float* __restrict__ norm_k, int rot, T* __restrict__ q_out,
                                              const PagedCache& cache, const int32_t* __restrict__ row_slot, int row, int pos,
                                              int head, int q_heads, float eps, int write_kv,
                                              const float* __restrict__ cs_tab, const float* __restrict__ sn_tab) {
    const int lane = threadIdx.x & 31;
    const int hd = cache.head_dim, half = rot >> 1;
    const int q_dim = q_heads * hd, kv_dim = cache.kv_heads * hd;
    const bool is_q = head < q_heads;
    const int kh = is_q ? 0 : head - q_heads;
    if (!is_q && !write_kv) return;
    const T* src = qkv + (int64_t)row * (q_dim + 2 * kv_dim) + (is_q ? head * hd : q_dim + kh * hd);
    const float* nw = is_q ? norm_q : norm_k;

    T* dst;
    if (is_q) {
        dst = q_out + (int64_t)row * q_dim + head * hd;
    } else {
        const int64_t off = cache_row_offset(cache, row_slot[row], pos, kh, 0);
        if (off < 0) return;
        dst = (T*)cache.base + off;
    }

    // The common shape (whole head rotated, head_dim a multiple of 4 up to 256): each lane owns the
    // pairs (i, i + half) for i = 2 lane, 2 lane + 1 (+ 64 ...), keeps them in registers between the
    // sum of squares and the rotation, and moves two values per access.
    if (rot == hd && (hd & 3) == 0 && hd <= 256) {
        float a[2][2], b[2][2];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int i = 2 * lane + 64 * it;
            if (i < half) {
                load2(src + i, a[it]);
                load2(src + i + half, b[it]);
                ss += a[it][0] * a[it][0] + a[it][1] * a[it][1] + b[it][0] * b[it][0] + b[it][1] * b[it][1];
            }
        }
        float scale = 1.f;
        if (nw) {
            ss = warp_sum(ss);
            scale = 1.0f / sqrtf(ss / (float)hd + eps);
        }
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int i = 2 * lane + 64 * it;
            if (i < half) {
                float ra[2], rb[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float x = a[it][e], y = b[it][e];
                    if (nw) {
                        x = x * scale * nw[i + e];
                        y = y * scale * nw[i + e + half];
                    }
                    const float sn = sn_tab[i + e], cs = cs_tab[i + e];
                    ra[e] = x * cs - y * sn;
                    rb[e] = y * cs + x * sn;
                }
                store2(dst + i, ra);
                store2(dst + i + half, rb);
            }
        }
        if (!is_q) {
            const T* vs = src + kv_dim;
            T* vd = dst + (int64_t)cache.kv_heads * cache.page_size * hd;
            for (int i = 2 * lane; i < hd; i += 64) copy2(vd + i, vs + i);
        }
        return;
    }

    float scale = 1.f;
    if (nw) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) {
            const float x = to_f32(src[i]);
            ss += x * x;
        }
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    for (int i = lane; i < half; i += 32) {
        float a = to_f32(src[i]), b = to_f32(src[i + half]);
        if (nw) {
            a = a * scale * nw[i];
            b = b * scale * nw[i + half];
        }
        const float s = sn_tab[i], c = cs_tab[i];
        dst[i] = from_f32<T>(a * c - b * s);
        dst[i + half] = from_f32<T>(b * c + a * s);
    }
    for (int i = rot + lane; i < hd; i += 32) {
        float a = to_f32(src[i]);
        if (nw) a = a * scale * nw[i];
        dst[i] = from_f32<T>(a);
    }
    if (!is_q) {
        const T* vs = src + kv_dim;
        T* vd = dst + (int64_t)cache.kv_heads * cache.page_size * hd;
        for (int i = lane; i < hd; i += 32) vd[i] = vs[i];
    }
}


template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(const T* __restrict__ qkv, const float* __restrict__ norm_q,
                                             const float* __restrict__ norm_k,
                                             const float* __restrict__ inv_freq, int rot, T* __restrict__ q_out,
                                             PagedCache cache, const int32_t* __restrict__ row_slot,
                                             const int32_t* __restrict__ row_pos, int n_rows, int q_heads,
                                             float eps, int write_kv, const float* __restrict__ rope_table,
                                             int table_positions) {
    extern __shared__ float rope_cs[];          // [warps][rot]: per warp, cosines then sines (only without a table)
    pdl_prologue();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = q_heads + cache.kv_heads;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (int64_t)n_rows * heads) return;
    const int row = (int)(item / heads), head = (int)(item % heads);
    const int half = rot >> 1;
    const int pos = row_pos[row];
    // The row's cosines and sines: from the table the position encoding made at start-up
    // ([position][cos..., sin...]) when it covers the position, else computed here by the warp.
    const float* cs_tab;
    const float* sn_tab;
    if (rope_table != nullptr && pos >= 0 && pos < table_positions) {
        cs_tab = rope_table + (int64_t)pos * rot;
        sn_tab = cs_tab + half;
    } else {
        float* c = rope_cs + warp * rot;
        float* sn = c + half;
        for (int i = lane; i < half; i += 32) sincosf((float)pos * inv_freq[i], &sn[i], &c[i]);
        __syncwarp();
        cs_tab = c;
        sn_tab = sn;
    }
    rope_one_head<T>(qkv, norm_q, norm_k, rot, q_out, cache, row_slot, row, pos, head, q_heads, eps, write_kv, cs_tab, sn_tab);
}

// The same for the common shapes (whole head rotated, head_dim 32, 64, 128 or 256, a table for the
// row's position): head_dim / 16 lanes per head, each owning 8 consecutive values of the first half
// and the 8 they pair with, moved 16 bytes at a time; a warp serves 512 / head_dim heads at once.
template <typename T, int HD>
__global__ void qk_norm_rope_kv_write_vec_kernel(const T* __restrict__ qkv, const float* __restrict__ norm_q,
                                                 const float* __restrict__ norm_k, T* __restrict__ q_out,
                                                 PagedCache cache, const int32_t* __restrict__ row_slot,
                                                 const int32_t* __restrict__ row_pos, int n_rows, int q_heads, float eps,
                                                 int write_kv, const float* __restrict__ rope_table, int table_positions,
                                                 const float* __restrict__ inv_freq) {
    constexpr int LPH = HD / 16;        // lanes per head
    constexpr int HPW = 32 / LPH;       // heads per warp
    constexpr int HALF = HD / 2;
    // Positions, slots, the page table, the norm weights and the rotation table are older than any
    // kernel still running; only q|k|v comes from the kernel before this one.  So everything but
    // q|k|v is asked for before the wait: the end of the product is followed by one trip to memory.
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int heads = q_heads + cache.kv_heads;
    const int64_t item = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * HPW + lane / LPH;
    const bool live = item < (int64_t)n_rows * heads;
    const int row = live ? (int)(item / heads) : 0, head = live ? (int)(item % heads) : 0;
    const int c = (lane % LPH) * 8;     // this lane's values: c .. c + 7 and HALF + c .. HALF + c + 7
    const int q_dim = q_heads * HD, kv_dim = cache.kv_heads * HD;
    const bool is_q = head < q_heads;
    const int kh = is_q ? 0 : head - q_heads;
    const T* src = qkv + (int64_t)row * (q_dim + 2 * kv_dim) + (is_q ? head * HD : q_dim + kh * HD);
    const float* nw = is_q ? norm_q : norm_k;
    const int pos = row_pos[row];
    const bool writes = live && (is_q || write_kv);
    T* dst = nullptr;
    if (writes) {
        if (is_q) {
            dst = q_out + (int64_t)row * q_dim + head * HD;
        } else {
            const int64_t off = cache_row_offset(cache, row_slot[row], pos, kh, 0);
            if (off >= 0) dst = (T*)cache.base + off;
        }
    }
    float wa[8], wb[8], cs[8], sn[8];
    if (nw) {
        load8(nw + c, wa);
        load8(nw + HALF + c, wb);
    }
    if (pos >= 0 && pos < table_positions) {
        load8(rope_table + (int64_t)pos * HD + c, cs);
        load8(rope_table + (int64_t)pos * HD + HALF + c, sn);
    } else {        // a position the table does not cover
#pragma unroll
        for (int k = 0; k < 8; ++k) sincosf((float)pos * inv_freq[c + k], &sn[k], &cs[k]);
    }
    pdl_wait();
    float a[8], b[8];
    load8(src + c, a);
    load8(src + HALF + c, b);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += a[k] * a[k] + b[k] * b[k];
#pragma unroll
    for (int o = 1; o < LPH; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (dst == nullptr) return;
    if (nw) {
        const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            a[k] = a[k] * scale * wa[k];
            b[k] = b[k] * scale * wb[k];
        }
    }
    float ra[8], rb[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        ra[k] = a[k] * cs[k] - b[k] * sn[k];
        rb[k] = b[k] * cs[k] + a[k] * sn[k];
    }
    store8(dst + c, ra);
    store8(dst + HALF + c, rb);
    if (!is_q) {
        const T* vs = src + kv_dim;
        T* vd = dst + (int64_t)cache.kv_heads * cache.page_size * HD;
        copy16(vd + c, vs + c);
        copy16(vd + HALF + c, vs + HALF + c);
    }
}

template <typename T>
static int launch_rope_vec(const T* qkv, const float* norm_q, const float* norm_k, T* q_out, const PagedCache& cache,
                           const int32_t* row_slot, const int32_t* row_pos, int n_rows, int q_heads, float eps, int write_kv,
                           const float* rope_table, int table_positions, const float* inv_freq, cudaStream_t stream) {
    const int hd = cache.head_dim;
    const int64_t items = (int64_t)n_rows * (q_heads + cache.kv_heads);
    const int hpw = 32 / (hd / 16), warps = 4;
    const int64_t blocks = (items + (int64_t)hpw * warps - 1) / ((int64_t)hpw * warps);
    X0NE_REQUIRE(blocks <= 0x7fffffff, "rope: too many rows");
#define X0NE_ROPE_VEC(HDV)                                                                                             \
    x0ne_launch(qk_norm_rope_kv_write_vec_kernel<T, HDV>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, qkv, norm_q, \
                norm_k, q_out, cache, row_slot, row_pos, n_rows, q_heads, eps, write_kv, rope_table, table_positions, inv_freq)
    if (hd == 32) X0NE_ROPE_VEC(32);
    else if (hd == 64) X0NE_ROPE_VEC(64);
    else if (hd == 128) X0NE_ROPE_VEC(128);
    else X0NE_ROPE_VEC(256);
#undef X0NE_ROPE_VEC
    X0NE_LAUNCH_CHECK();
}

X0NE_API int x0ne_qk_norm_rope_kv_write(const void* qkv, int dt, const float* norm_q, const float* norm_k,
                                        const float* inv_freq, int rotary_dim, void* q_out, PagedCache cache,
                                        const int32_t* row_slot, const int32_t* row_pos, int n_rows, int q_heads,
                                        float eps, int write_kv, const float* rope_table, int table_positions,
                                        cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && q_heads > 0 && cache.kv_heads > 0 && cache.head_dim > 0, "rope: bad sizes");
    X0NE_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= cache.head_dim,
                 "rope: rotary_dim %d must be even and at most head_dim %d", rotary_dim, cache.head_dim);
    X0NE_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "rope: no inv_freq table");
    if (n_rows == 0) return 0;
    const int hd_ = cache.head_dim;
    if (rope_table != nullptr && rotary_dim == hd_ && (hd_ == 32 || hd_ == 64 || hd_ == 128 || hd_ == 256) &&
        (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache.base | (uintptr_t)rope_table | (uintptr_t)norm_q |
          (uintptr_t)norm_k) & 15) == 0) {
        if (dt == X0NE_F32)
            return launch_rope_vec<float>((const float*)qkv, norm_q, norm_k, (float*)q_out, cache, row_slot, row_pos, n_rows,
                                          q_heads, eps, write_kv, rope_table, table_positions, inv_freq, stream);
        if (dt == X0NE_BF16)
            return launch_rope_vec<bf16>((const bf16*)qkv, norm_q, norm_k, (bf16*)q_out, cache, row_slot, row_pos, n_rows,
                                         q_heads, eps, write_kv, rope_table, table_positions, inv_freq, stream);
    }
    // one warp per (row, head)
    const int heads = q_heads + cache.kv_heads;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * heads;
    X0NE_REQUIRE((items + warps - 1) / warps <= 0x7fffffff, "rope: too many rows");
    const dim3 grid((unsigned)((items + warps - 1) / warps));
    const size_t smem = (size_t)warps * rotary_dim * sizeof(float);
    if (dt == X0NE_F32)
        x0ne_launch(qk_norm_rope_kv_write_kernel<float>, dim3(grid), dim3(warps * 32), smem, stream, 
            (const float*)qkv, norm_q, norm_k, inv_freq, rotary_dim, (float*)q_out, cache, row_slot, row_pos, n_rows,
            q_heads, eps, write_kv, rope_table, table_positions);
    else if (dt == X0NE_BF16)
        x0ne_launch(qk_norm_rope_kv_write_kernel<bf16>, dim3(grid), dim3(warps * 32), smem, stream, 
            (const bf16*)qkv, norm_q, norm_k, inv_freq, rotary_dim, (bf16*)q_out, cache, row_slot, row_pos, n_rows,
            q_heads, eps, write_kv, rope_table, table_positions);
    else
        X0NE_REQUIRE(false, "rope: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// SwiGLU on the packed [gate; up] row: out[i] = T(g / (1 + expf(-g)) * u)
// (x0ne-core/kernels/cuda/swiglu.cu:5-11).
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (i >= inter) return;
    const T* row = gate_up + (int64_t)r * 2 * inter;
    const float g = to_f32(row[i]), u = to_f32(row[inter + i]);
    out[(int64_t)r * inter + i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// 8 values per thread with 16-byte accesses (inter % 8 == 0 and aligned rows).
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int64_t total8) {
    pdl_prologue();
    const int per_row = inter / 8;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total8; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = e / per_row;
        const int i = (int)(e % per_row) * 8;
        const T* row = gate_up + r * 2 * inter;
        float g[8], u[8], o[8];
        load8(row + i, g);
        load8(row + inter + i, u);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.0f + expf(-g[k])) * u[k];
        store8(out + r * inter + i, o);
    }
}

X0NE_API int x0ne_swiglu(const void* gate_up, void* out, int dt, int n_rows, int inter, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && inter > 0, "swiglu: rows %d inter %d", n_rows, inter);
    if (n_rows == 0) return 0;
    X0NE_REQUIRE(n_rows <= 65535 * 1024, "swiglu: too many rows for one launch");
    const int esize = dt == X0NE_F32 ? 4 : 2;
    if (inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0 && ((int64_t)inter * esize) % 16 == 0) {
        const int64_t total8 = (int64_t)n_rows * (inter / 8);
        int64_t blocks = (total8 + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        if (dt == X0NE_F32)
            x0ne_launch(swiglu_vec_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out, inter, total8);
        else if (dt == X0NE_BF16)
            x0ne_launch(swiglu_vec_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total8);
        else
            X0NE_REQUIRE(false, "swiglu: unknown dtype tag %d", dt);
        X0NE_LAUNCH_CHECK();
    }
    for (int r0 = 0; r0 < n_rows; r0 += 65535) {
        const int nr = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
        dim3 grid((inter + 255) / 256, nr);
        if (dt == X0NE_F32)
            x0ne_launch(swiglu_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)gate_up + (int64_t)r0 * 2 * inter,
                        (float*)out + (int64_t)r0 * inter, inter);
        else if (dt == X0NE_BF16)
            x0ne_launch(swiglu_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)gate_up + (int64_t)r0 * 2 * inter,
                        (bf16*)out + (int64_t)r0 * inter, inter);
        else
            X0NE_REQUIRE(false, "swiglu: unknown dtype tag %d", dt);
    }
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Embedding: resid[r] = f32(table[tokens[r]]); an id outside the table gives a zero row
// (x0ne-core/kernels/cuda/embedding.cu:5-17).  The engine there copies the row and lets the
// first add-norm add it to a zeroed residual (x0ne-core/runtime/src/engine.rs:744-745); here
// the row is written straight into the float32 residual, which is the same value.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ tokens,
                                 float* __restrict__ resid, int hidden, int vocab) {
    pdl_prologue();
    const int row = blockIdx.x;
    const int t = tokens[row];
    float* dst = resid + (int64_t)row * hidden;
    if (t < 0 || t >= vocab) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const T* src = table + (int64_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]);
}

// The same with 16-byte accesses (hidden % 8 == 0, aligned rows): all of a row's loads are in flight
// at once, where the loop above waits for memory once per 256 values (9.5 us for 8 rows of 4,096).
template <typename T>
__global__ void embedding_vec_kernel(const T* __restrict__ table, const int32_t* __restrict__ tokens,
                                     float* __restrict__ resid, int hidden, int vocab) {
    pdl_prologue();
    const int row = blockIdx.x;
    const int t = tokens[row];
    float* dst = resid + (int64_t)row * hidden;
    const bool none = t < 0 || t >= vocab;
    const T* src = table + (int64_t)(none ? 0 : t) * hidden;
    for (int i0 = threadIdx.x * 8; i0 < hidden; i0 += 4 * blockDim.x * 8) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x * 8;
            if (i < hidden && !none) load8(src + i, v[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x * 8;
            if (i < hidden) {
                if (none) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[u][k] = 0.f;
                }
                store8(dst + i, v[u]);
            }
        }
    }
}

X0NE_API int x0ne_embedding(const void* table, int dt, const int32_t* tokens, float* resid, int n_rows,
                            int hidden, int vocab, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && hidden > 0 && vocab > 0, "embedding: rows %d hidden %d vocab %d", n_rows, hidden, vocab);
    if (n_rows == 0) return 0;
    const int block = hidden >= 1024 ? 256 : 128;
    if (hidden % 8 == 0 && (((uintptr_t)table | (uintptr_t)resid) & 15) == 0 && (dt == X0NE_F32 || dt == X0NE_BF16)) {
        const int threads = hidden / 8 >= 256 ? 256 : (hidden / 8 + 31) / 32 * 32;
        if (dt == X0NE_F32)
            x0ne_launch(embedding_vec_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)table, tokens, resid, hidden, vocab);
        else
            x0ne_launch(embedding_vec_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, (const bf16*)table, tokens, resid, hidden, vocab);
        X0NE_LAUNCH_CHECK();
    }
    if (dt == X0NE_F32)
        x0ne_launch(embedding_kernel<float>, dim3(n_rows), dim3(block), 0, stream, (const float*)table, tokens, resid, hidden, vocab);
    else if (dt == X0NE_BF16)
        x0ne_launch(embedding_kernel<bf16>, dim3(n_rows), dim3(block), 0, stream, (const bf16*)table, tokens, resid, hidden, vocab);
    else
        X0NE_REQUIRE(false, "embedding: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

