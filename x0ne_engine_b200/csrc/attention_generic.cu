// Attention over the paged cache, any head size, any window: the plain kernel.
//
// It serves the 32-bit path for prefill and decode alike, and the bfloat16 path for shapes the
// tensor-core kernels do not take.  One warp per (query row, q head).  The query at position p
// of sequence slot s reads keys max(0, p - window + 1) .. p of that slot (causal by loop bound,
// no mask matrix: x0ne-core/kernels/cuda/attention.cu:21,28,102-103); q head h reads kv head
// h / (q_heads / kv_heads) (attention.cu:20).  Online softmax in float32
// (attention.cu:44-59,138-157): running max m, sum l, p_j = expf(s_j - m_new),
// alpha = expf(m - m_new), acc = acc * alpha + sum p_j v_j, out = acc / l.
//
// The order of every sum depends only on the query's position and the window: keys are taken
// in tiles of 32 starting at the first visible key, lane t owns key t of the tile, each score
// is one sequential dot product, the tile's sum is an xor-shuffle tree, and the values are
// accumulated key by key.  So the same query gives the same bits whether it arrives in a
// prompt, in a later chunk, alone or in a batch.
#include "common.cuh"

#define ATT_MAX_I 8  // head_dim <= 32 * ATT_MAX_I

template <typename T>
__global__ void attention_rows_kernel(const T* __restrict__ q, T* __restrict__ out, PagedCache cache,
                                      const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                      int n_rows, int q_heads, float scale, int window) {
    extern __shared__ float smem[];
    pdl_prologue();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int hd = cache.head_dim;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + w;
    if (item >= (int64_t)n_rows * q_heads) return;
    const int row = (int)(item / q_heads), head = (int)(item % q_heads);
    const int kh = head / (q_heads / cache.kv_heads);
    const int pos = row_pos[row], slot = row_slot[row];
    float* qs = smem + w * hd;
    const T* qr = q + ((int64_t)row * q_heads + head) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qr[d]) * scale;
    __syncwarp();

    const int j_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int64_t v_off = (int64_t)cache.kv_heads * cache.page_size * hd;
    const T* base = (const T*)cache.base;
    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_I];
#pragma unroll
    for (int i = 0; i < ATT_MAX_I; ++i) acc[i] = 0.f;

    for (int j0 = j_lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        int64_t off = -1;
        float s = -INFINITY;
        if (j <= pos) {
            off = cache_row_offset(cache, slot, j, kh, 0);
            if (off >= 0) {
                const T* kr = base + off;
                float a = 0.f;
                for (int d = 0; d < hd; ++d) a = fmaf(qs[d], to_f32(kr[d]), a);
                s = a;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;  // no readable key in this tile
        const float p = off >= 0 ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < ATT_MAX_I; ++i) acc[i] *= alpha;
        const int nt = min(32, pos - j0 + 1);
        for (int t = 0; t < nt; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const long long ot = __shfl_sync(0xffffffffu, (long long)off, t);
            if (ot < 0) continue;
            const T* vr = base + ot + v_off;
#pragma unroll
            for (int i = 0; i < ATT_MAX_I; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pt, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    T* o = out + ((int64_t)row * q_heads + head) * hd;
    const float inv = l > 0.f ? 1.0f / l : 0.f;      // a row with no readable key (a padding row) gets zeros
#pragma unroll
    for (int i = 0; i < ATT_MAX_I; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = from_f32<T>(acc[i] * inv);
    }
}

X0NE_API int x0ne_attention_rows(const void* q, void* out, int dt, PagedCache cache, const int32_t* row_slot,
                                 const int32_t* row_pos, int n_rows, int q_heads, float scale, int window,
                                 cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && q_heads > 0 && cache.kv_heads > 0 && q_heads % cache.kv_heads == 0,
                 "attention: %d q heads over %d kv heads", q_heads, cache.kv_heads);
    X0NE_REQUIRE(cache.head_dim > 0 && cache.head_dim <= 32 * ATT_MAX_I,
                 "attention: head_dim %d is beyond the plain kernel's limit of %d", cache.head_dim, 32 * ATT_MAX_I);
    X0NE_REQUIRE(window >= 0, "attention: negative window");
    if (n_rows == 0) return 0;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * q_heads;
    const unsigned grid = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * cache.head_dim * sizeof(float);
    if (dt == X0NE_F32)
        x0ne_launch(attention_rows_kernel<float>, dim3(grid), dim3(warps * 32), smem, stream, (const float*)q, (float*)out, cache, row_slot,
                                                                       row_pos, n_rows, q_heads, scale, window);
    else if (dt == X0NE_BF16)
        x0ne_launch(attention_rows_kernel<bf16>, dim3(grid), dim3(warps * 32), smem, stream, (const bf16*)q, (bf16*)out, cache, row_slot,
                                                                      row_pos, n_rows, q_heads, scale, window);
    else
        X0NE_REQUIRE(false, "attention: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}
