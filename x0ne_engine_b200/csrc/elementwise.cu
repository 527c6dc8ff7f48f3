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

X0NE_API int x0ne_embedding(const void* table, int dt, const int32_t* tokens, float* resid, int n_rows,
                            int hidden, int vocab, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && hidden > 0 && vocab > 0, "embedding: rows %d hidden %d vocab %d", n_rows, hidden, vocab);
    if (n_rows == 0) return 0;
    const int block = hidden >= 1024 ? 256 : 128;
    if (dt == X0NE_F32)
        x0ne_launch(embedding_kernel<float>, dim3(n_rows), dim3(block), 0, stream, (const float*)table, tokens, resid, hidden, vocab);
    else if (dt == X0NE_BF16)
        x0ne_launch(embedding_kernel<bf16>, dim3(n_rows), dim3(block), 0, stream, (const bf16*)table, tokens, resid, hidden, vocab);
    else
        X0NE_REQUIRE(false, "embedding: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Residual add, then RMSNorm: r = resid + f32(delta) (one IEEE add, stored back);
// out = T(r * rsqrt(mean(r^2) + eps) * w)  (x0ne-core/kernels/cuda/rmsnorm.cu:11-20; eps is
// inside the root; the weight multiplies directly).  `delta` may be null (norm only).
// `rows`, if given, lists the source rows to process; output row i then belongs to source row
// rows[i] (used to norm only the rows whose logits are wanted).
// One block per row; the sum of squares is a fixed-order block sum.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ out,
                                   const int32_t* __restrict__ rows, int hidden, float eps) {
    __shared__ float sh[32];
    pdl_prologue();
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = resid + src * hidden;
    const T* d = delta ? delta + src * hidden : nullptr;
    T* o = out + (int64_t)blockIdx.x * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = r[i];
        if (d) {
            v = v + to_f32(d[i]);
            r[i] = v;
        }
        ss += v * v;
    }
    const float total = block_sum(ss, sh);
    const float scale = 1.0f / sqrtf(total / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(r[i] * scale * w[i]);
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
__device__ __forceinline__ void copy2(float* d, const float* s) { *reinterpret_cast<float2*>(d) = *reinterpret_cast<const float2*>(s); }
__device__ __forceinline__ void copy2(bf16* d, const bf16* s) { *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(s); }

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ out,
                                       const int32_t* __restrict__ rows, int hidden, float eps) {
    __shared__ float sh[32];
    pdl_prologue();
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = resid + src * hidden;
    const T* d = delta ? delta + src * hidden : nullptr;
    T* o = out + (int64_t)blockIdx.x * hidden;
    float v[VEC_IT][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < VEC_IT; ++it) {
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
    for (int it = 0; it < VEC_IT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 8;
        if (i < hidden) {
            float wv[8], ov[8];
            load8(w + i, wv);
#pragma unroll
            for (int k = 0; k < 8; ++k) ov[k] = v[it][k] * scale * wv[k];
            store8(o + i, ov);
        }
    }
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
            x0ne_launch(add_rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, resid, (const float*)delta, w, (float*)out, rows, hidden, eps);
        else if (dt == X0NE_BF16)
            x0ne_launch(add_rmsnorm_vec_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, resid, (const bf16*)delta, w, (bf16*)out, rows, hidden, eps);
        else
            X0NE_REQUIRE(false, "add_rmsnorm: unknown dtype tag %d", dt);
        X0NE_LAUNCH_CHECK();
    }
    const int block = 256;
    if (dt == X0NE_F32)
        x0ne_launch(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(block), 0, stream, resid, (const float*)delta, w, (float*)out, rows, hidden, eps);
    else if (dt == X0NE_BF16)
        x0ne_launch(add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(block), 0, stream, resid, (const bf16*)delta, w, (bf16*)out, rows, hidden, eps);
    else
        X0NE_REQUIRE(false, "add_rmsnorm: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Per-head RMSNorm of q and k (optional), rotate-half RoPE, and the K/V write into the
// paged cache (x0ne-core/kernels/cuda/rope.cu:7-47).  One block per row: the row's sines and cosines
// are computed once into shared memory, then one warp per head; heads
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
    extern __shared__ float rope_cs[];          // [half] cosines, then [half] sines of this row's angles
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int heads = q_heads + cache.kv_heads;
    const int row = blockIdx.x;
    const int hd = cache.head_dim, half = rot >> 1;
    const int q_dim = q_heads * hd, kv_dim = cache.kv_heads * hd;
    const int pos = row_pos[row];
    // The row's cosines and sines: from the table the position encoding made at start-up
    // ([position][cos..., sin...]) when it covers the position, else computed here.
    const float* cs_tab;
    const float* sn_tab;
    if (rope_table != nullptr && pos >= 0 && pos < table_positions) {
        cs_tab = rope_table + (int64_t)pos * rot;
        sn_tab = cs_tab + half;
    } else {
        float* c = rope_cs;
        float* sn = rope_cs + half;
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &c[i]);
        __syncthreads();
        cs_tab = c;
        sn_tab = sn;
    }
    // blockIdx.y picks this block's share of the heads (one share when there are many rows)
    const int per_block = (heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per_block, h_hi = min(heads, h_lo + per_block);
    for (int head = h_lo + (threadIdx.x >> 5); head < h_hi; head += blockDim.x >> 5)
        rope_one_head<T>(qkv, norm_q, norm_k, rot, q_out, cache, row_slot, row, pos, head, q_heads, eps, write_kv, cs_tab, sn_tab);
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
    // One block of 8 warps per row when there are many rows; with few rows (decode) the heads of a
    // row are spread over several blocks of 4 warps, each of which computes the row's table itself.
    const int heads = q_heads + cache.kv_heads;
    const int warps = n_rows >= 64 ? 8 : 4;
    const int shares = n_rows >= 64 ? 1 : (heads + warps - 1) / warps;
    X0NE_REQUIRE(n_rows <= 0x7fffffff && shares <= 65535, "rope: too many rows or heads");
    const dim3 grid((unsigned)n_rows, (unsigned)shares);
    const size_t smem = (size_t)rotary_dim * sizeof(float);
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
