// bfloat16 attention over the paged cache on the tensor cores: a varlen causal flash kernel for
// passes that bring several tokens per sequence, and a split-KV flash-decoding kernel for passes
// that bring one.
//
// What they compute is what the plain kernel computes (attention_generic.cu; formulas from
// x0ne-core/kernels/cuda/attention.cu:20-59,138-157,165-171,257-269): q head h reads kv head
// h / (q_heads / kv_heads); the query at position p sees keys max(0, p - window + 1) .. p; scores,
// running max, exponentials, sums and the output accumulator are float32; one rounding to
// bfloat16 at the end.  Scores are kept in the log2 domain (scale * log2 e folded into one
// multiply, exp2f for the exponentials).
//
// Both kernels take key tiles of one cache page (64 positions) at a time: a page of one kv head
// is one contiguous block of 64 x head_dim values, copied to shared memory with 16-byte
// cp.async, rows padded by 16 bytes so that ldmatrix reads are free of bank conflicts.
// Tensor-core path: mma.sync m16n8k16 (bf16 in, f32 accumulate).
// head_dim: any multiple of 16 up to 128 (template); other shapes use the plain kernel.
#include "common.cuh"

#define PAGE 64
#define PADE 8  // padding elements per shared-memory row (16 bytes)
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies rows [0, PAGE) of one page of one kv head (K or V) into padded shared memory; rows whose
// position is past `last_pos` are zero-filled (a page's tail may never have been written).
template <int HD, int THREADS>
__device__ __forceinline__ void load_page_tile(bf16* dst, const bf16* src, int first_pos, int last_pos, int tid) {
    constexpr int CH = HD / 8;  // 16-byte chunks per row
#pragma unroll
    for (int c = tid; c < PAGE * CH; c += THREADS) {
        const int r = c / CH, k = c % CH;
        bf16* d = dst + r * (HD + PADE) + k * 8;
        if (src != nullptr && first_pos + r <= last_pos)
            cp_async16(d, src + r * HD + k * 8);
        else
            *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
}

__device__ __forceinline__ const bf16* page_ptr(const PagedCache& c, int slot, int logical_page, int kv_head, int which) {
    const int page = c.page_table[(int64_t)slot * c.table_stride + (logical_page % c.ring_pages)];
    if (page < 0 || page >= c.n_pages) return nullptr;
    return (const bf16*)c.base + (int64_t)page * c.page_stride +
           ((int64_t)which * c.kv_heads + kv_head) * c.page_size * c.head_dim;
}

// One warp: S(16 x 16*NT8/2 keys) = Q(16 x HD) K^T from a padded K tile, keys [key0, key0 + 8*NT8).
template <int HD, int NT8>
__device__ __forceinline__ void qk_tile(float (*s)[4], const uint32_t (*qf)[4], const bf16* ks, int key0, int lane) {
#pragma unroll
    for (int n = 0; n < NT8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < NT8 / 2; ++n2) {
            uint32_t b0, b1, b2, b3;
            const int row = key0 + n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int col = kk * 16 + (((lane >> 3) & 1) << 3);
            ldsm_x4(b0, b1, b2, b3, ks + row * (HD + PADE) + col);
            mma_bf16(s[2 * n2], qf[kk], b0, b1);
            mma_bf16(s[2 * n2 + 1], qf[kk], b2, b3);
        }
    }
}

// One warp: O(16 x HD) += P(16 x 8*NT8 keys) V from a padded V tile, keys [key0, key0 + 8*NT8).
template <int HD, int NT8>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*s)[4], const bf16* vs, int key0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NT8 / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
            uint32_t b0, b1, b2, b3;
            const int row = key0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int col = n2 * 16 + ((lane >> 4) << 3);
            ldsm_x4_t(b0, b1, b2, b3, vs + row * (HD + PADE) + col);
            mma_bf16(o[2 * n2], a, b0, b1);
            mma_bf16(o[2 * n2 + 1], a, b2, b3);
        }
    }
}

// Online-softmax update of one warp's 16 rows with the scores s (already scaled to the log2 domain
// and masked with -inf); leaves p in s.
template <int HD, int NT8>
__device__ __forceinline__ void softmax_update(float (*s)[4], float (*o)[4], float* m, float* l) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < NT8; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * h], s[n][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[h], mx);
        const float base = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = exp2f(m[h] - base);
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < NT8; ++n) {
            s[n][2 * h] = exp2f(s[n][2 * h] - base);
            s[n][2 * h + 1] = exp2f(s[n][2 * h + 1] - base);
            sum += s[n][2 * h] + s[n][2 * h + 1];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[h] = l[h] * alpha + sum;
        m[h] = m_new;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            o[n][2 * h] *= alpha;
            o[n][2 * h + 1] *= alpha;
        }
    }
}

// ----------------------------------------------------------------------------------------
// Prefill: grid (q_heads, tiles); a tile is up to 64 * MT consecutive rows of one sequence.
// 4 warps, 16 * MT query rows each: with MT = 2 every K and V fragment read from shared memory
// feeds two MMAs, which is what the shared-memory bandwidth needs.  Q stays in shared memory.
// ----------------------------------------------------------------------------------------
struct PrefillArgs {
    const bf16* q;
    bf16* out;
    const int32_t* tile_seq;       // [tiles]
    const int32_t* tile_row0;      // [tiles] first row of the tile within the pass
    const int32_t* seq_first_row;  // [seqs + 1]
    const int32_t* seq_slot;       // [seqs]
    const int32_t* seq_pos0;       // [seqs] position of the sequence's first row in this pass
    int32_t q_heads;
    int32_t window;
    float scale_log2;
};

template <int HD, int MT>
__global__ void __launch_bounds__(128) attention_prefill_kernel(PrefillArgs a, PagedCache cache) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int LD = HD + PADE;
    constexpr int ROWS = 64 * MT;                   // query rows of a tile; a warp owns 16 * MT of them
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [ROWS][LD]
    bf16* ks = qs + ROWS * LD;                      // [2][64][LD]
    bf16* vs = ks + 2 * 64 * LD;                    // [2][64][LD]
    pdl_prologue();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the longest contexts (the last tiles of a sequence) are scheduled first
    const int head = blockIdx.x, tile = gridDim.y - 1 - blockIdx.y;
    const int kh = head / (a.q_heads / cache.kv_heads);
    const int seq = a.tile_seq[tile], row0 = a.tile_row0[tile];
    const int seq_end = a.seq_first_row[seq + 1];
    const int nrows = min(ROWS, seq_end - row0);
    const int slot = a.seq_slot[seq];
    const int pos_first = a.seq_pos0[seq] + (row0 - a.seq_first_row[seq]);
    const int pos_last = pos_first + nrows - 1;
    const int q_dim = a.q_heads * HD;

    // Q tile -> shared (rows past the tile's end are zero)
    constexpr int CH = HD / 8;
    for (int c = tid; c < ROWS * CH; c += 128) {
        const int r = c / CH, k = c % CH;
        bf16* d = qs + r * LD + k * 8;
        if (r < nrows)
            cp_async16(d, a.q + (int64_t)(row0 + r) * q_dim + head * HD + k * 8);
        else
            *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    const int j_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    const int kt_lo = j_lo / PAGE, kt_hi = pos_last / PAGE;
    // first K/V tile
    load_page_tile<HD, 128>(ks, page_ptr(cache, slot, kt_lo, kh, 0), kt_lo * PAGE, pos_last, tid);
    load_page_tile<HD, 128>(vs, page_ptr(cache, slot, kt_lo, kh, 1), kt_lo * PAGE, pos_last, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    const int wrow0 = warp * 16 * MT;               // this warp's first row in the tile
    float o[MT][HD / 8][4];
    float m[MT][2], l[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[t][n][i] = 0.f;
        m[t][0] = m[t][1] = -INFINITY;
        l[t][0] = l[t][1] = 0.f;
    }
    const int warp_first = pos_first + wrow0;
    const int warp_last = min(pos_last, warp_first + 16 * MT - 1);

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        if (kt + 1 <= kt_hi) {
            load_page_tile<HD, 128>(ks + (buf ^ 1) * 64 * LD, page_ptr(cache, slot, kt + 1, kh, 0), (kt + 1) * PAGE, pos_last, tid);
            load_page_tile<HD, 128>(vs + (buf ^ 1) * 64 * LD, page_ptr(cache, slot, kt + 1, kh, 1), (kt + 1) * PAGE, pos_last, tid);
        }
        cp_async_commit();
        const bf16* kb = ks + buf * 64 * LD;
        const bf16* vb = vs + buf * 64 * LD;
        // A warp whose rows all lie before this tile's first key has nothing to do here.
        if (kt * PAGE <= warp_last) {
            float s[MT][8][4];
#pragma unroll
            for (int t = 0; t < MT; ++t)
#pragma unroll
                for (int n = 0; n < 8; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s[t][n][i] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t kf[4][4];
#pragma unroll
                for (int n2 = 0; n2 < 4; ++n2) {
                    const int row = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    const int col = kk * 16 + (((lane >> 3) & 1) << 3);
                    ldsm_x4(kf[n2][0], kf[n2][1], kf[n2][2], kf[n2][3], kb + row * LD + col);
                }
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    uint32_t qf[4];
                    const int row = wrow0 + t * 16 + (lane & 15), col = kk * 16 + ((lane >> 4) << 3);
                    ldsm_x4(qf[0], qf[1], qf[2], qf[3], qs + row * LD + col);
#pragma unroll
                    for (int n2 = 0; n2 < 4; ++n2) {
                        mma_bf16(s[t][2 * n2], qf, kf[n2][0], kf[n2][1]);
                        mma_bf16(s[t][2 * n2 + 1], qf, kf[n2][2], kf[n2][3]);
                    }
                }
            }
            const bool edge = (kt * PAGE + PAGE - 1 > warp_first) ||
                              (a.window > 0 && kt * PAGE <= warp_last - a.window + 16 * MT);
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                const int p0 = warp_first + t * 16 + (lane >> 2);
#pragma unroll
                for (int n = 0; n < 8; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float v = s[t][n][i] * a.scale_log2;
                        if (edge) {
                            const int j = kt * PAGE + n * 8 + ((lane & 3) << 1) + (i & 1);
                            const int p = p0 + ((i >> 1) << 3);
                            if (j > p || (a.window > 0 && j <= p - a.window)) v = -INFINITY;
                        }
                        s[t][n][i] = v;
                    }
                softmax_update<HD, 8>(s[t], o[t], m[t], l[t]);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[MT][4];
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    pa[t][0] = pack_bf16(s[t][2 * kk][0], s[t][2 * kk][1]);
                    pa[t][1] = pack_bf16(s[t][2 * kk][2], s[t][2 * kk][3]);
                    pa[t][2] = pack_bf16(s[t][2 * kk + 1][0], s[t][2 * kk + 1][1]);
                    pa[t][3] = pack_bf16(s[t][2 * kk + 1][2], s[t][2 * kk + 1][3]);
                }
#pragma unroll
                for (int n2 = 0; n2 < HD / 16; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    const int col = n2 * 16 + ((lane >> 4) << 3);
                    ldsm_x4_t(b0, b1, b2, b3, vb + row * LD + col);
#pragma unroll
                    for (int t = 0; t < MT; ++t) {
                        mma_bf16(o[t][2 * n2], pa[t], b0, b1);
                        mma_bf16(o[t][2 * n2 + 1], pa[t], b2, b3);
                    }
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();
    }
    // write
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = wrow0 + t * 16 + (lane >> 2) + 8 * h;
            if (r < nrows) {
                const float inv = 1.0f / l[t][h];
                bf16* dst = a.out + (int64_t)(row0 + r) * q_dim + head * HD + ((lane & 3) << 1);
#pragma unroll
                for (int n = 0; n < HD / 8; ++n)
                    *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[t][n][2 * h] * inv, o[t][n][2 * h + 1] * inv);
            }
        }
}

// ----------------------------------------------------------------------------------------
// Decode: one query row per sequence.  grid (splits, kv_heads * group_chunks, sequences); a block
// serves up to 16 q heads of one kv head (they are the 16 rows of the MMA tile) over its share of
// the sequence's pages.  The 4 warps take 16 keys each of every 64-key page, each with its own
// running (m, l, o) and its own cp.async ring (no block barrier in the loop); they are merged in
// shared memory at the end, and the blocks of one
// (sequence, kv head) are merged by whichever of them finishes last, in the fixed order of the
// splits (the last-arriver scheme of x0ne-core/kernels/cuda/attention.cu:439-455: nobody waits).
// ----------------------------------------------------------------------------------------
struct DecodeArgs {
    const bf16* q;
    bf16* out;
    const int32_t* row_slot;
    const int32_t* row_pos;
    float* part_o;         // [rows * q_heads][parts][HD]
    float* part_ml;        // [rows * q_heads][parts][2]
    int32_t* counters;     // [rows * kv_heads * group_chunks], zero before the launch, zero after
    int32_t q_heads;
    int32_t window;
    int32_t splits;        // blocks per (sequence, kv head): the pages are cut into this many ranges
    float scale_log2;
    int32_t cluster_merge;  // the splits form thread-block clusters of splits / groups blocks that merge in shared memory
    int32_t groups;         // clusters per (sequence, kv head); more than one: their results meet in scratch
};

#define DEC_MAX_PAGES 128

// Shared memory of another block of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(const void* local, int rank) {
    uint32_t r;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_dsmem(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 ld_dsmem4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// CLUSTER: the blocks of one (sequence, kv head) form `groups` thread-block clusters of at most 8
// blocks, each of which merges its partial results through its blocks' shared memory; one cluster
// writes the output itself, several leave one partial result each in global scratch and the last
// block to arrive merges those (a long context at a small batch: 4 clusters of 8 put 256 blocks on
// 8 kv heads).  Not CLUSTER: every block's partial result goes through scratch.
// WARPS: 4, or 8 for launches whose blocks have an SM each (one sequence): the second four warps
// take every other page.  Inside a step the kernel starts early and has its first pages in shared
// memory when q arrives; what the step then waits for is each warp's chain of dependent
// instructions over its pages, and with 8 warps a warp has half as many.
template <int HD, int STAGES, bool CLUSTER, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) attention_decode_kernel(DecodeArgs a, PagedCache cache) {
    constexpr int THREADS = 32 * WARPS, NPAR = WARPS / 4;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int LD = HD + PADE;
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [16][LD]
    bf16* ks = qs + 16 * LD;                        // [WARPS][STAGES][K, V][16][LD]: each warp's own ring
    __shared__ int s_last;
    // What the kernel before this one (the q/k-norm + RoPE + cache write of this step) produced is q
    // and the newest row of the cache.  Positions, slots, the page table and all older rows are
    // older than that, so the first slices are requested before waiting for it.
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kq = warp & 3, par = warp >> 2;       // which 16 keys of a page, and which pages (every NPAR-th from par)
    const int split = blockIdx.x, b = blockIdx.z;
    const int csize = CLUSTER ? a.splits / a.groups : 1;        // blocks of one cluster
    const int crank = CLUSTER ? split % csize : 0;
    const int parts = CLUSTER ? a.groups : a.splits;            // partial results that meet in scratch
    const int part = CLUSTER ? split / csize : split;
    const int G = a.q_heads / cache.kv_heads;
    const int gchunks = (G + 15) / 16;
    const int kh = blockIdx.y / gchunks, gc = blockIdx.y % gchunks;
    const int head0 = kh * G + gc * 16;
    const int nheads = min(16, G - gc * 16);
    const int slot = a.row_slot[b], pos = a.row_pos[b];
    const int q_dim = a.q_heads * HD;

    constexpr int CH = HD / 8;
    const int j_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int pg_first = j_lo / PAGE, pg_count = pos / PAGE - pg_first + 1;
    const int p_lo = pg_first + (int)(((int64_t)pg_count * split) / a.splits);
    const int p_hi = pg_first + (int)(((int64_t)pg_count * (split + 1)) / a.splits);   // exclusive
    const int n_pages = p_hi - p_lo;

    // The page numbers of this block's range, read once (a lookup inside the loop would put a
    // dependent global load in front of every copy).
    __shared__ int s_page[DEC_MAX_PAGES];
    for (int i = tid; i < n_pages && i < DEC_MAX_PAGES; i += THREADS) {
        const int pg = cache.page_table[(int64_t)slot * cache.table_stride + ((p_lo + i) % cache.ring_pages)];
        s_page[i] = (pg >= 0 && pg < cache.n_pages) ? pg : -1;
    }
    __syncthreads();
    const int64_t head_off = (int64_t)kh * cache.page_size * cache.head_dim;
    const int64_t v_off = (int64_t)cache.kv_heads * cache.page_size * cache.head_dim;
    auto tile_ptr = [&](int i) -> const bf16* {
        int pg;
        if (i < DEC_MAX_PAGES) {
            pg = s_page[i];
        } else {
            pg = cache.page_table[(int64_t)slot * cache.table_stride + ((p_lo + i) % cache.ring_pages)];
            if (pg >= cache.n_pages) pg = -1;
        }
        return pg < 0 ? nullptr : (const bf16*)cache.base + (int64_t)pg * cache.page_stride + head_off;
    };

    // Each warp streams its own 16 keys of its pages (K and V rows 16 kq .. 16 kq + 15) through a
    // private ring of STAGES slots: no block-wide barrier inside the loop, STAGES - 1 slices in flight.
    const int my_pages = n_pages > par ? (n_pages - par + NPAR - 1) / NPAR : 0;
    bf16* wring = ks + warp * STAGES * 2 * 16 * LD;
    auto load_slice = [&](int st, int j) {
        const int i = par + NPAR * j;
        const bf16* kp = tile_ptr(i);
        bf16* kd = wring + (st * 2) * 16 * LD;
        bf16* vd = kd + 16 * LD;
        const int first_pos = (p_lo + i) * PAGE + kq * 16;
#pragma unroll
        for (int c = lane; c < 16 * CH; c += 32) {
            const int r = c / CH, k = c % CH;
            if (kp != nullptr && first_pos + r <= pos) {
                const bf16* src = kp + (kq * 16 + r) * HD + k * 8;
                cp_async16(kd + r * LD + k * 8, src);
                cp_async16(vd + r * LD + k * 8, src + v_off);
            } else {
                *reinterpret_cast<uint4*>(kd + r * LD + k * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + r * LD + k * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    bool waited = false;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < my_pages) {
            if (!waited && (p_lo + par + NPAR * s + 1) * PAGE > pos) {    // the page that holds the newest row
                pdl_wait();
                waited = true;
            }
            load_slice(s, s);
        }
        cp_async_commit();
    }
    if (!waited) pdl_wait();
    for (int c = tid; c < 16 * CH; c += THREADS) {
        const int r = c / CH, k = c % CH;
        bf16* d = qs + r * LD + k * 8;
        if (r < nheads)
            cp_async16(d, a.q + (int64_t)b * q_dim + (head0 + r) * HD + k * 8);
        else
            *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    uint32_t qf[HD / 16][4];

    cp_async_wait<0>();  // the first slices and q (q is the last group of the prologue)
    __syncthreads();     // q was copied by all warps
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = lane & 15, col = kk * 16 + ((lane >> 4) << 3);
        ldsm_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + row * LD + col);
    }
    for (int it = 0; it < my_pages; ++it) {
        if (it > 0) {
            cp_async_wait<STAGES - 2>();
            __syncwarp();        // the slice was copied by all lanes of this warp; all have left the last one
        }
        {   // refill the slot that was consumed in the previous iteration
            const int nx = it + STAGES - 1;
            if (nx < my_pages) load_slice(nx % STAGES, nx);
            cp_async_commit();
        }
        const bf16* kb = wring + ((it % STAGES) * 2) * 16 * LD;
        const bf16* vb = kb + 16 * LD;
        const int first_pos = (p_lo + par + NPAR * it) * PAGE + kq * 16;
        if (first_pos <= pos) {
            float s[2][4];
            qk_tile<HD, 2>(s, qf, kb, 0, lane);
            const bool edge = (first_pos + 15 > pos) || (a.window > 0 && first_pos < j_lo);
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = s[n][i] * a.scale_log2;
                    if (edge) {
                        const int j = first_pos + n * 8 + ((lane & 3) << 1) + (i & 1);
                        if (j > pos || j < j_lo) v = -INFINITY;
                    }
                    s[n][i] = v;
                }
            softmax_update<HD, 2>(s, o, m, l);
            pv_tile<HD, 2>(o, s, vb, 0, lane);
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the warps through shared memory (the K/V stages are free now).  Rows of the group that
    // hold no head are not written; a row takes HD + 8 floats, so that the rows of a warp's
    // fragment fall into different banks; every thread then merges four consecutive values
    // (1.3-1.9 us of a launch went to this step when it wrote all 16 rows value by value).
    constexpr int MOS = HD + 8;
    float* mo = reinterpret_cast<float*>(ks);            // [WARPS][16][MOS]
    float* mml = mo + WARPS * 16 * MOS;                  // [WARPS][16][2]
    float* xml = mml + WARPS * 16 * 2;                   // [16][2]: this block's (m, l) for the cluster; its o is mo[0]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + 8 * h;
        if (r < nheads) {
#pragma unroll
            for (int n = 0; n < HD / 8; ++n)
                *reinterpret_cast<float2*>(mo + (warp * 16 + r) * MOS + n * 8 + ((lane & 3) << 1)) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
            if ((lane & 3) == 0) {
                mml[(warp * 16 + r) * 2] = m[h];
                mml[(warp * 16 + r) * 2 + 1] = l[h];
            }
        }
    }
    __syncthreads();
    const int64_t qrow0 = (int64_t)b * a.q_heads + head0;
    for (int e = tid; e < nheads * (HD / 4); e += THREADS) {
        const int r = e / (HD / 4), d = (e % (HD / 4)) * 4;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = mml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + r) * MOS + d);
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
            L += mml[(w * 16 + r) * 2 + 1] * f;
        }
        if (a.splits == 1) {
            *reinterpret_cast<uint2*>(a.out + (qrow0 + r) * HD + d) =
                make_uint2(pack_bf16(acc.x / L, acc.y / L), pack_bf16(acc.z / L, acc.w / L));
        } else if (CLUSTER) {
            *reinterpret_cast<float4*>(mo + r * MOS + d) = acc;      // over the first warp's values of the same elements, which only this thread read
            if (d == 0) {
                xml[r * 2] = M;
                xml[r * 2 + 1] = L;
            }
        } else {
            *reinterpret_cast<float4*>(a.part_o + ((qrow0 + r) * parts + part) * HD + d) = acc;
            if (d == 0) {
                a.part_ml[((qrow0 + r) * parts + part) * 2] = M;
                a.part_ml[((qrow0 + r) * parts + part) * 2 + 1] = L;
            }
        }
    }
    if (a.splits == 1) return;
    if constexpr (CLUSTER) {
        // Every block of the cluster takes a share of the output and sums the cluster's splits in their order.
        cluster_sync_all();
        for (int e = crank * THREADS + tid; e < nheads * (HD / 4); e += THREADS * csize) {
            const int r = e / (HD / 4), d = (e % (HD / 4)) * 4;
            float M = -INFINITY;
            for (int sp = 0; sp < csize; ++sp) M = fmaxf(M, ld_dsmem(dsmem_addr(xml + r * 2, sp)));
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp = 0; sp < csize; ++sp) {
                const float ms = ld_dsmem(dsmem_addr(xml + r * 2, sp));
                const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
                L += ld_dsmem(dsmem_addr(xml + r * 2 + 1, sp)) * f;
                const float4 v = ld_dsmem4(dsmem_addr(mo + r * MOS + d, sp));
                acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
            }
            if (parts == 1) {
                const float il = 1.0f / L;
                bf16* dst = a.out + (qrow0 + r) * HD + d;
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * il, acc.y * il), pack_bf16(acc.z * il, acc.w * il));
            } else {
                // this cluster's result, not yet divided by its sum, for the merge of the clusters
                *reinterpret_cast<float4*>(a.part_o + ((qrow0 + r) * parts + part) * HD + d) = acc;
                if (d == 0) {
                    a.part_ml[((qrow0 + r) * parts + part) * 2] = M;
                    a.part_ml[((qrow0 + r) * parts + part) * 2 + 1] = L;
                }
            }
        }
        cluster_sync_all();      // nobody leaves while its shared memory may still be read
        if (parts == 1) return;
    }

    // The last block to arrive (every block of every cluster counts itself in) merges the partial
    // results in their fixed order.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int32_t* cnt = a.counters + ((int64_t)b * cache.kv_heads * gchunks + blockIdx.y);
        const int prev = atomicAdd(cnt, 1);
        s_last = prev == (int)gridDim.x - 1;
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (parts <= 8) {
        // Few parts: every thread asks for all it needs at once (the parts' maxima and sums of its
        // row, and its four output values of every part), so the merge is one trip to L2; the sums
        // are taken in the order of the parts, as below.
        for (int e = tid; e < nheads * (HD / 4); e += THREADS) {
            const int r = e / (HD / 4), d = (e % (HD / 4)) * 4;
            const float2* pml = reinterpret_cast<const float2*>(a.part_ml + (qrow0 + r) * parts * 2);
            const float* po = a.part_o + (qrow0 + r) * parts * HD + d;
            float2 ml[8];
            float4 v[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
                if (sp < parts) {
                    ml[sp] = __ldcg(pml + sp);
                    v[sp] = __ldcg(reinterpret_cast<const float4*>(po + sp * HD));
                }
            float M = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
                if (sp < parts) M = fmaxf(M, ml[sp].x);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
                if (sp < parts) {
                    const float f = ml[sp].x == -INFINITY ? 0.f : exp2f(ml[sp].x - M);
                    L += ml[sp].y * f;
                    acc.x += v[sp].x * f; acc.y += v[sp].y * f; acc.z += v[sp].z * f; acc.w += v[sp].w * f;
                }
            const float il = 1.0f / L;
            bf16* dst = a.out + (qrow0 + r) * HD + d;
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * il, acc.y * il), pack_bf16(acc.z * il, acc.w * il));
        }
        return;
    }
    // Per (head, part) weights first, all loads in parallel, then every thread sums four
    // consecutive output values over the parts in their order.
    float* wgt = reinterpret_cast<float*>(ks);           // [16][parts]: exp2(m_s - M); then [16]: 1 / L
    float* inv_l = wgt + 16 * parts;
    for (int e = tid; e < nheads * parts; e += THREADS) {
        const int r = e / parts, sp = e % parts;
        wgt[r * parts + sp] = __ldcg(a.part_ml + ((qrow0 + r) * parts + sp) * 2);
    }
    __syncthreads();
    if (tid < nheads) {
        float M = -INFINITY;
        for (int sp = 0; sp < parts; ++sp) M = fmaxf(M, wgt[tid * parts + sp]);
        float L = 0.f;
        for (int sp = 0; sp < parts; ++sp) {
            const float ms = wgt[tid * parts + sp];
            const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
            wgt[tid * parts + sp] = f;
            L += __ldcg(a.part_ml + ((qrow0 + tid) * parts + sp) * 2 + 1) * f;
        }
        inv_l[tid] = 1.0f / L;
    }
    __syncthreads();
    for (int e = tid; e < nheads * (HD / 4); e += THREADS) {
        const int r = e / (HD / 4), d = (e % (HD / 4)) * 4;
        const float* po = a.part_o + (qrow0 + r) * parts * HD + d;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int sp = 0; sp < parts; ++sp) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(po + sp * HD));
            const float f = wgt[r * parts + sp];
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        const float il = inv_l[r];
        bf16* dst = a.out + (qrow0 + r) * HD + d;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * il, acc.y * il), pack_bf16(acc.z * il, acc.w * il));
    }
}

// ----------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------
#define PREFILL_MT 2
template <int HD>
static int launch_prefill(const PrefillArgs& a, const PagedCache& cache, int n_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)(64 * PREFILL_MT + 4 * 64) * (HD + PADE) * sizeof(bf16);
    static OncePerDevice configured;
    if (configured.need()) {
        cudaFuncSetAttribute(attention_prefill_kernel<HD, PREFILL_MT>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD, PREFILL_MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            x0ne_set_error("attention_prefill: cannot set %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured.done();
    }
    dim3 grid(a.q_heads, n_tiles);
    x0ne_launch(attention_prefill_kernel<HD, PREFILL_MT>, dim3(grid), dim3(128), smem, stream, a, cache);
    X0NE_LAUNCH_CHECK();
}

#define DECODE_STAGES 3
#define DECODE_CLUSTER_MAX 8      // the largest cluster every launch may ask for
#define DECODE_WIDE_WARPS 8       // warps of a block that has an SM to itself

template <int HD, int WARPS>
static size_t decode_smem_bytes() {
    size_t smem = (size_t)(16 + WARPS * DECODE_STAGES * 2 * 16) * (HD + PADE) * sizeof(bf16);
    const size_t merge = (size_t)(WARPS * 16 * (HD + 8) + WARPS * 16 * 2 + 16 * 2) * sizeof(float);
    if (smem < 16 * (HD + PADE) * sizeof(bf16) + merge) smem = 16 * (HD + PADE) * sizeof(bf16) + merge;
    return smem;
}

// How many clusters of `cluster` blocks of the kernel with this many warps run at once; 0 if unknown.
template <int HD, int WARPS>
static int decode_clusters_at_once(int cluster) {
    const size_t smem = decode_smem_bytes<HD, WARPS>();
    auto kernel = attention_decode_kernel<HD, DECODE_STAGES, true, WARPS>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1024, 1);
    cfg.blockDim = dim3(32 * WARPS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

template <int HD, bool CLUSTER, int WARPS>
static int launch_decode_variant(const DecodeArgs& a, const PagedCache& cache, int n_rows, cudaStream_t stream) {
    const size_t smem = decode_smem_bytes<HD, WARPS>();
    static OncePerDevice configured;
    if (configured.need()) {
        cudaFuncSetAttribute(attention_decode_kernel<HD, DECODE_STAGES, CLUSTER, WARPS>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, DECODE_STAGES, CLUSTER, WARPS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            x0ne_set_error("attention_decode: cannot set %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured.done();
    }
    const int G = a.q_heads / cache.kv_heads;
    dim3 grid(a.splits, cache.kv_heads * ((G + 15) / 16), n_rows);
    if (CLUSTER)
        x0ne_launch_clusters(attention_decode_kernel<HD, DECODE_STAGES, CLUSTER, WARPS>, dim3(grid), dim3(32 * WARPS), a.splits / a.groups,
                             smem, stream, a, cache);
    else
        x0ne_launch(attention_decode_kernel<HD, DECODE_STAGES, CLUSTER, WARPS>, dim3(grid), dim3(32 * WARPS), smem, stream, a, cache);
    X0NE_LAUNCH_CHECK();
}

template <int HD>
static int launch_decode(const DecodeArgs& a, const PagedCache& cache, int n_rows, cudaStream_t stream) {
    const int cluster = a.splits / a.groups;
    if (a.cluster_merge && a.splits > 1 && cluster <= DECODE_CLUSTER_MAX) {
        // Eight warps per block where all clusters of the launch then still run at once (one block
        // per SM: one sequence of a model with 8 kv heads); asked of the runtime once per device
        // and cluster size.
        static int wide_fit[64][DECODE_CLUSTER_MAX + 1];
        static OncePerDevice asked[DECODE_CLUSTER_MAX + 1];
        const int dev = OncePerDevice::device();
        if (dev >= 0 && decode_smem_bytes<HD, DECODE_WIDE_WARPS>() <= 227 * 1024) {
            if (asked[cluster].need()) {
                wide_fit[dev][cluster] = decode_clusters_at_once<HD, DECODE_WIDE_WARPS>(cluster);
                asked[cluster].done();
            }
            const int G = a.q_heads / cache.kv_heads;
            const int64_t clusters = (int64_t)n_rows * cache.kv_heads * ((G + 15) / 16) * a.groups;
            if (clusters <= wide_fit[dev][cluster])
                return launch_decode_variant<HD, true, DECODE_WIDE_WARPS>(a, cache, n_rows, stream);
        }
        return launch_decode_variant<HD, true, 4>(a, cache, n_rows, stream);
    }
    return launch_decode_variant<HD, false, 4>(a, cache, n_rows, stream);
}

#define DISPATCH_HD(HDV, CALL)                     \
    switch (HDV) {                                 \
        case 16: { constexpr int HD_ = 16; CALL; } \
        case 32: { constexpr int HD_ = 32; CALL; } \
        case 48: { constexpr int HD_ = 48; CALL; } \
        case 64: { constexpr int HD_ = 64; CALL; } \
        case 80: { constexpr int HD_ = 80; CALL; } \
        case 96: { constexpr int HD_ = 96; CALL; } \
        case 112: { constexpr int HD_ = 112; CALL; } \
        case 128: { constexpr int HD_ = 128; CALL; } \
        default: break;                            \
    }

static int check_common(const PagedCache& cache, int q_heads, const char* what) {
    X0NE_REQUIRE(cache.page_size == PAGE, "%s: pages of %d positions, the kernel takes %d", what, cache.page_size, PAGE);
    X0NE_REQUIRE(cache.head_dim % 16 == 0 && cache.head_dim >= 16 && cache.head_dim <= 128,
                 "%s: head_dim %d is not a multiple of 16 between 16 and 128 (use the plain kernel)", what, cache.head_dim);
    X0NE_REQUIRE(q_heads > 0 && cache.kv_heads > 0 && q_heads % cache.kv_heads == 0, "%s: %d q heads over %d kv heads",
                 what, q_heads, cache.kv_heads);
    return 0;
}

X0NE_API int x0ne_attention_prefill_bf16(const void* q, void* out, PagedCache cache, const int32_t* tile_seq,
                                         const int32_t* tile_row0, int n_tiles, const int32_t* seq_first_row,
                                         const int32_t* seq_slot, const int32_t* seq_pos0, int q_heads, float scale,
                                         int window, cudaStream_t stream) {
    if (int e = check_common(cache, q_heads, "attention_prefill")) return e;
    X0NE_REQUIRE(n_tiles >= 0 && n_tiles <= 65535, "attention_prefill: %d tiles in one launch (limit 65535)", n_tiles);
    X0NE_REQUIRE(window >= 0, "attention_prefill: negative window");
    if (n_tiles == 0) return 0;
    PrefillArgs a{(const bf16*)q, (bf16*)out, tile_seq, tile_row0, seq_first_row, seq_slot, seq_pos0, q_heads, window,
                  scale * LOG2E};
    DISPATCH_HD(cache.head_dim, return launch_prefill<HD_>(a, cache, n_tiles, stream));
    X0NE_REQUIRE(false, "attention_prefill: head_dim %d not built", cache.head_dim);
}

// Rows of one tile of the prefill kernel: callers build their tile tables with it.
X0NE_API int x0ne_attention_prefill_tile_rows() { return 64 * PREFILL_MT; }

// Blocks of the decode kernel that fit on one SM at head_dim 128 (shared memory decides): callers
// size `splits` so that a launch is one wave.
X0NE_API int x0ne_attention_decode_blocks_per_sm() { return DECODE_STAGES <= 2 ? 3 : (DECODE_STAGES == 3 ? 2 : 1); }

// How many clusters of `splits` blocks of the decode kernel the GPU holds at once (they do not pack
// its GPCs completely, so this is less than resident blocks / splits); 0 if unknown.  Callers keep
// (sequences x kv heads x group chunks) within it so that a launch is one wave.
template <int HD>
static int decode_max_clusters(int splits) {
    return decode_clusters_at_once<HD, 4>(splits);
}

X0NE_API int x0ne_attention_decode_max_clusters(int head_dim, int splits) {
    if (splits < 1 || splits > DECODE_CLUSTER_MAX) return 0;
    DISPATCH_HD(head_dim, return decode_max_clusters<HD_>(splits));
    return 0;
}

// Scratch the decode kernel needs for `n_rows` sequences with `splits` splits, in bytes:
// partial outputs, partial (m, l), and the arrival counters (which must start at zero).
X0NE_API int64_t x0ne_attention_decode_scratch_bytes(int n_rows, int q_heads, int kv_heads, int head_dim, int splits) {
    const int G = q_heads / kv_heads, gchunks = (G + 15) / 16;
    const int64_t po = (int64_t)n_rows * q_heads * splits * head_dim * 4;
    const int64_t ml = (int64_t)n_rows * q_heads * splits * 2 * 4;
    const int64_t cn = (int64_t)n_rows * kv_heads * gchunks * 4;
    return po + ml + ((cn + 255) / 256) * 256;
}

// `groups` = 1: `splits` blocks per (sequence, kv head); without scratch (and with at most 8 splits)
// they are one thread-block cluster and merge in shared memory, with scratch every block leaves its
// partial result there and the last one merges.  `groups` > 1: `groups` clusters of splits / groups
// blocks (2 to 8) each; a cluster merges in shared memory, the clusters' results meet in scratch
// (sized by x0ne_attention_decode_scratch_bytes for `groups` parts).
static int decode_entry(const void* q, void* out, PagedCache cache, const int32_t* row_slot, const int32_t* row_pos,
                        int n_rows, int q_heads, float scale, int window, int splits, int groups, void* scratch,
                        int64_t scratch_bytes, cudaStream_t stream) {
    if (int e = check_common(cache, q_heads, "attention_decode")) return e;
    X0NE_REQUIRE(n_rows >= 0 && n_rows <= 65535, "attention_decode: %d rows in one launch (limit 65535)", n_rows);
    X0NE_REQUIRE(splits >= 1 && splits <= 64, "attention_decode: %d splits (1 to 64)", splits);
    X0NE_REQUIRE(groups >= 1 && splits % groups == 0 && (groups == 1 || (splits / groups >= 2 && splits / groups <= DECODE_CLUSTER_MAX)),
                 "attention_decode: %d splits in %d clusters (clusters of 2 to %d blocks)", splits, groups, DECODE_CLUSTER_MAX);
    X0NE_REQUIRE(window >= 0, "attention_decode: negative window");
    if (n_rows == 0) return 0;
    DecodeArgs a{};
    a.q = (const bf16*)q;
    a.out = (bf16*)out;
    a.row_slot = row_slot;
    a.row_pos = row_pos;
    a.q_heads = q_heads;
    a.window = window;
    a.splits = splits;
    a.groups = groups;
    a.scale_log2 = scale * LOG2E;
    if (groups == 1 && splits > 1 && scratch == nullptr && splits <= DECODE_CLUSTER_MAX) {
        a.cluster_merge = 1;      // no scratch given: the splits of a (sequence, kv head) merge inside their cluster
    } else if (splits > 1) {
        const int parts = groups > 1 ? groups : splits;
        const int64_t need = x0ne_attention_decode_scratch_bytes(n_rows, q_heads, cache.kv_heads, cache.head_dim, parts);
        X0NE_REQUIRE(scratch != nullptr && scratch_bytes >= need, "attention_decode: scratch of %lld bytes, %lld needed",
                     (long long)scratch_bytes, (long long)need);
        const int G = q_heads / cache.kv_heads, gchunks = (G + 15) / 16;
        const int64_t cn = (((int64_t)n_rows * cache.kv_heads * gchunks * 4 + 255) / 256) * 256;
        a.counters = (int32_t*)scratch;
        a.part_o = (float*)((char*)scratch + cn);            // 256-byte aligned: read back as float4
        a.part_ml = a.part_o + (int64_t)n_rows * q_heads * parts * cache.head_dim;
        a.cluster_merge = groups > 1;
        X0NE_REQUIRE(((uintptr_t)scratch & 15) == 0, "attention_decode: scratch is not 16-byte aligned");
    }
    DISPATCH_HD(cache.head_dim, return launch_decode<HD_>(a, cache, n_rows, stream));
    X0NE_REQUIRE(false, "attention_decode: head_dim %d not built", cache.head_dim);
}

X0NE_API int x0ne_attention_decode_bf16(const void* q, void* out, PagedCache cache, const int32_t* row_slot,
                                        const int32_t* row_pos, int n_rows, int q_heads, float scale, int window,
                                        int splits, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    return decode_entry(q, out, cache, row_slot, row_pos, n_rows, q_heads, scale, window, splits, 1, scratch, scratch_bytes, stream);
}

X0NE_API int x0ne_attention_decode_grouped_bf16(const void* q, void* out, PagedCache cache, const int32_t* row_slot,
                                                const int32_t* row_pos, int n_rows, int q_heads, float scale, int window,
                                                int splits, int groups, void* scratch, int64_t scratch_bytes,
                                                cudaStream_t stream) {
    return decode_entry(q, out, cache, row_slot, row_pos, n_rows, q_heads, scale, window, splits, groups, scratch, scratch_bytes,
                        stream);
}
