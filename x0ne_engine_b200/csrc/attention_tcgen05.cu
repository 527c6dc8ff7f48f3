// Causal GQA flash attention for passes with many rows, on the 5th-generation tensor cores:
// both products of a tile (S = Q K^T and P V) are tcgen05.mma with their results in tensor memory,
// Q and the cache pages come to shared memory by TMA, and the softmax runs in registers, two
// threads per query row.  Same arithmetic as the mma.sync kernel of attention_bf16.cu (formulas:
// x0ne-core/kernels/cuda/attention.cu:20-59,138-157): scores, maximum and sum, exponentials
// and the output accumulator in float32, P rounded to bfloat16 for the second product, one
// rounding of the output at the end.  head_dim 64 or 128; other sizes use the mma.sync kernel.
//
// A block takes one tile of up to 128 query rows of one sequence and one q head (grid: q heads x
// tiles, longest contexts first) and walks the cache pages (64 keys) the tile can see:
//   * QK warp (warp 8): TMA loads of Q (once) and of each page's K tile (two stages, 128-byte
//     swizzle; a page of one kv head is 64 consecutive rows of the cache seen as one long
//     [rows, head_dim] matrix); issues S(i) = Q K(i)^T (M 128, N 64, K 16 x head_dim/16) into one of
//     two score buffers in tensor memory as soon as the softmax threads have read that buffer, so
//     the scores of page i + 1 are computed while page i is in the softmax.
//   * PV warp (warp 9): TMA loads of the V tiles (two stages); when the softmax threads have
//     written P(i) it issues O += P(i) V(i) (M 128, N head_dim, K 16 x 4; V is the N-major operand,
//     straight from the page as it lies in the cache).
//     Both warps run their loops with all lanes and let one elected lane issue; every lane comes
//     back together (__syncwarp) before any of them waits for what that lane had to ask for.
//   * softmax threads (warps 0-7; warps w and w + 4 share rows 32 (w % 4) ... + 31 and take one
//     half of a page's keys each): read S from tensor memory, mask, agree on the row's reference
//     maximum, and write P = 2^((s - reference) * scale) to shared memory in the swizzled layout
//     the MMA reads.  The output accumulates in tensor memory across the pages (the MMA adds to
//     it); it is rescaled there, by the softmax threads, only when a row's maximum has grown by
//     more than 2^8 over its reference, and divided by the row's sum at the end.
// Every barrier wait is bounded; when one runs out the block records it in `status`, skips the
// rest, frees its tensor memory and returns.  Two blocks fit on an SM and overlap each other.
#include "tcgen05.cuh"

struct AttnTcArgs {
    bf16* out;
    const int32_t* tile_seq;       // [tiles]
    const int32_t* tile_row0;      // [tiles] first row of the tile within the pass
    const int32_t* seq_first_row;  // [seqs + 1]
    const int32_t* seq_slot;       // [seqs]
    const int32_t* seq_pos0;       // [seqs]
    int32_t q_heads;
    int32_t window;
    float scale_log2;
};

struct AttnTcShared {
    uint64_t q_full;
    uint64_t k_full[2];
    uint64_t v_full[2];
    uint64_t s_ready[2];
    uint64_t s_free[2];        // the softmax threads have read a score buffer
    uint64_t p_ready;
    uint64_t pv_ready;
    uint64_t pair[4];          // the two warps that share 32 rows meet here
    uint32_t tmem_base;
    int failed;
    __nv_bfloat16 xmax[2][128];   // each half's row maxima, for the other half (512 bytes; at the end: 128 floats)
};

// N-major (the matrix's N runs along the 128-byte rows) shared-memory descriptor, 128-byte swizzle:
// 8-row groups 1024 bytes apart, 64-wide column blocks `block_bytes` apart.
__device__ __forceinline__ uint64_t tc_desc_nmajor(uint32_t smem_addr, uint32_t block_bytes) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (((block_bytes >> 4) & 0x3FFFu) << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
}
// The running maximum a row's exponentials refer to is only raised when the new maximum exceeds it
// by more than this many powers of two: then the accumulator in tensor memory has to be rescaled,
// which is a read-modify-write of the whole row.  Until then p = 2^(s - reference) stays below 2^8.
#define ATC_RESCALE_LOG2 8.0f

#define ATC_THREADS 320      // 8 softmax warps (4 row groups x 2 column halves), the QK warp and the PV warp
#define ATC_TMEM_COLS 256

#ifdef X0NE_ATC_TIMING
__device__ long long atc_timing[32];
#define ATC_T(idx) do { if (timed) { const long long now_ = clock64(); atomicAdd((unsigned long long*)&atc_timing[idx], (unsigned long long)(now_ - t_last)); t_last = now_; } } while (0)
extern "C" __attribute__((visibility("default"))) int x0ne_atc_timing(long long* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, atc_timing, sizeof(atc_timing));
    long long zero[32] = {0};
    cudaMemcpyToSymbol(atc_timing, zero, sizeof(zero));
    return 0;
}
#else
#define ATC_T(idx) do { } while (0)
#endif

template <int HD>
__global__ void __launch_bounds__(ATC_THREADS, 2) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                           const __grid_constant__ CUtensorMap map_kv,
                                                                           AttnTcArgs a, PagedCache cache, int* status) {
    extern __shared__ __align__(1024) unsigned char atc_raw[];
    constexpr int NB = HD / 64;                   // 64-wide blocks of a head: 128 bytes per row each
    constexpr int Q_BYTES = NB * 128 * 128;       // [NB][128 rows][128 B]
    constexpr int KV_BYTES = NB * 64 * 128;       // one K or V tile: [NB][64 keys][128 B]
    constexpr int P_BYTES = 128 * 128;            // [128 rows][64 keys]
    unsigned char* qs = atc_raw;
    unsigned char* ks = qs + Q_BYTES;             // 2 stages
    unsigned char* vs = ks + 2 * KV_BYTES;        // 2 stages
    unsigned char* ps = vs + 2 * KV_BYTES;
    AttnTcShared* sh = reinterpret_cast<AttnTcShared*>(ps + P_BYTES);
    // the warp index through a shuffle, so that the compiler knows it is the same for the whole warp
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

    const int head = blockIdx.x, tile = gridDim.y - 1 - blockIdx.y;
    const int kh = head / (a.q_heads / cache.kv_heads);
    const int seq = a.tile_seq[tile], row0 = a.tile_row0[tile];
    const int nrows = min(128, a.seq_first_row[seq + 1] - row0);
    const int slot = a.seq_slot[seq];
    const int pos_first = a.seq_pos0[seq] + (row0 - a.seq_first_row[seq]);
    const int pos_last = pos_first + nrows - 1;
    const int j_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    const int kt_lo = j_lo / 64, n_kt = pos_last / 64 - kt_lo + 1;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(&sh->q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh->k_full[b], 1);
            mbar_init(&sh->v_full[b], 1);
            mbar_init(&sh->s_ready[b], 1);
            mbar_init(&sh->s_free[b], 256);
        }
        mbar_init(&sh->p_ready, 256);
        for (int b = 0; b < 4; ++b) mbar_init(&sh->pair[b], 64);
        mbar_init(&sh->pv_ready, 1);
        sh->failed = (tc_smem(atc_raw) & 1023u) != 0 ? 1 : 0;      // the swizzle needs 1024-byte aligned tiles
        if (sh->failed) atomicOr(status, 1 << 9);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)),
                     "r"(ATC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;       // S: two buffers of 64 columns; O: HD columns

    // The two control warps run their loops with all lanes (the values are the same in every lane,
    // which lets the compiler keep descriptors and addresses in uniform registers); one elected
    // lane issues the copies and the products.
    if (warp >= 8) {
        uint32_t leader = 0;
        asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
        // Page numbers are looked up well before the copies that need them (the table is older
        // than the kernel before this one): a lookup in front of a copy would be a dependent
        // global load in the loop.
        auto page_of = [&](int i) -> int {
            if (i >= n_kt) return 0;
            const int pg = cache.page_table[(int64_t)slot * cache.table_stride + ((kt_lo + i) % cache.ring_pages)];
            return (pg < 0 || pg >= cache.n_pages) ? 0 : pg;      // never out of range for a sequence that holds its pages
        };
        const int pg0 = page_of(0), pg1 = page_of(1);
        int pg_cur = page_of(2);
        bool ok = !sh->failed;
        auto wait = [&](uint64_t* bar, int parity, int code) {
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, status, code));
        };
        pdl_wait();      // q and the newest cache rows were written by the kernel before this one
        if (warp == 8) {
            // ---- scores: Q once, K pages through two stages, S(i) = Q K(i)^T into buffer i & 1
            auto load_k = [&](int i, int page) {
                const int st = i & 1;
                const int krow = ((page * 2 + 0) * cache.kv_heads + kh) * 64;
                if (leader) {
                    mbar_expect_tx(&sh->k_full[st], KV_BYTES);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
                        tma_load_2d(ks + st * KV_BYTES + nb * 64 * 128, &map_kv, nb * 64, krow, &sh->k_full[st]);
                }
                __syncwarp();      // no lane waits for what the elected lane has not yet asked for
            };
            if (leader && ok) {
                mbar_expect_tx(&sh->q_full, Q_BYTES);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) tma_load_2d(qs + nb * 128 * 128, &map_q, head * HD + nb * 64, row0, &sh->q_full);
            }
            __syncwarp();
            if (ok) {
                load_k(0, pg0);
                if (n_kt > 1) load_k(1, pg1);
            }
            // instruction descriptor: f32 accumulate, bf16 operands, M = 128, N = 64
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t qb = tc_smem(qs);
            wait(&sh->q_full, 0, 5);
            for (int i = 0; i < n_kt && ok; ++i) {
                const int st = i & 1;
                const int pg_next = page_of(i + 2);
                wait(&sh->k_full[st], (i >> 1) & 1, 6);
                if (i >= 2) wait(&sh->s_free[st], ((i - 2) >> 1) & 1, 12);      // the softmax of page i - 2 has read this buffer
                if (!ok) break;
                tc_fence_after();
                if (leader) {
                    const uint32_t kb = tc_smem(ks + st * KV_BYTES);
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk)
                        tc_mma(tmem_s + st * 64, tc_desc(qb + (kk / 4) * 128 * 128 + (kk % 4) * 32),
                               tc_desc(kb + (kk / 4) * 64 * 128 + (kk % 4) * 32), idesc_qk, kk > 0 ? 1u : 0u);
                    tc_commit(&sh->s_ready[st]);
                }
                __syncwarp();
                if (i >= 1 && i + 1 < n_kt) {      // K(i - 1) has been read when S(i - 1) is complete: its stage takes K(i + 1)
                    wait(&sh->s_ready[st ^ 1], ((i - 1) >> 1) & 1, 17);
                    if (!ok) break;
                    load_k(i + 1, pg_cur);
                }
                if (i >= 1) pg_cur = pg_next;
            }
        } else {
            // ---- output: V pages through two stages, O += P(i) V(i) when the softmax threads have written P(i)
            auto load_v = [&](int i, int page) {
                const int st = i & 1;
                const int vrow = ((page * 2 + 1) * cache.kv_heads + kh) * 64;
                if (leader) {
                    mbar_expect_tx(&sh->v_full[st], KV_BYTES);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
                        tma_load_2d(vs + st * KV_BYTES + nb * 64 * 128, &map_kv, nb * 64, vrow, &sh->v_full[st]);
                }
                __syncwarp();
            };
            if (ok) {
                load_v(0, pg0);
                if (n_kt > 1) load_v(1, pg1);
            }
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (((uint32_t)HD >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t pb = tc_smem(ps);
            for (int i = 0; i < n_kt && ok; ++i) {
                const int st = i & 1;
                const int pg_next = page_of(i + 3);
                wait(&sh->v_full[st], (i >> 1) & 1, 13);
                wait(&sh->p_ready, i & 1, 7);
                if (!ok) break;
                tc_fence_after();
                if (leader) {
                    const uint32_t vb = tc_smem(vs + st * KV_BYTES);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        tc_mma(tmem_o, tc_desc(pb + kk * 32), tc_desc_nmajor(vb + kk * 16 * 128, 64 * 128), idesc_pv,
                               (i > 0 || kk > 0) ? 1u : 0u);          // the output accumulates in tensor memory over the pages
                    tc_commit(&sh->pv_ready);
                }
                __syncwarp();
                if (i + 2 < n_kt) {       // V's stage is free once this product is done
                    wait(&sh->pv_ready, i & 1, 8);
                    if (!ok) break;
                    load_v(i + 2, pg_cur);
                }
                pg_cur = pg_next;
            }
        }
        if (!ok) sh->failed = 1;
    } else {
        // Two threads per row: warp w and warp w + 4 own rows 32 (w % 4) ... + 31 (their lanes of
        // tensor memory) and each takes one half of a page's 64 keys, and one half of the output's
        // columns.  They agree on the row's reference maximum through shared memory.
        const int sw = warp & 3, half = warp >> 2;
        const int r = sw * 32 + lane;
        const int p = pos_first + r;
        const uint32_t lane_base = (uint32_t)(sw * 32) << 16;
        const float sc = a.scale_log2;
        float m_ref = -INFINITY, l = 0.f;                     // reference maximum (raw scores) and this half's sum of p
        int pair_phase = 0;
        bool ok = !sh->failed;
#ifdef X0NE_ATC_TIMING
        const bool timed = blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
        long long t_last = clock64();
#endif
        for (int i = 0; i < n_kt && ok; ++i) {
            const int kt = kt_lo + i;
            if (!(ok = mbar_wait(&sh->s_ready[i & 1], (i >> 1) & 1, status, 10))) break;
            ATC_T(0);
            tc_fence_after();
            float s[32];
            tc_ld32(tmem_s + (i & 1) * 64 + half * 32 + lane_base, s);
            tc_fence_before();
            mbar_arrive(&sh->s_free[i & 1]);      // the scores are in registers: the buffer may take the page after next
            ATC_T(1);
            const bool edge = (kt * 64 + 63 > pos_first) || (a.window > 0 && kt * 64 <= pos_last - a.window);
            if (edge) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int j = kt * 64 + half * 32 + c;
                    if (j > p || (a.window > 0 && j <= p - a.window)) s[c] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains instead of one
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], s[c + e]);
            }
            // The halves exchange their maxima rounded up to bfloat16 (a reference may lie above the
            // true maximum; it must only be the same for the whole row).
            const __nv_bfloat16 mine = __float2bfloat16_ru(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            // The other half must have read the maximum of the page before, and the scores come a
            // page ahead, so nothing else orders that: every thread reads it before it arrives on
            // p_ready, so wait for that phase (it completes about when this thread arrived itself).
            if (i > 0 && !(ok = mbar_wait(&sh->p_ready, (i - 1) & 1, status, 18))) break;
            sh->xmax[half][r] = mine;
            mbar_arrive(&sh->pair[sw]);
            ATC_T(2);
            if (!(ok = mbar_wait(&sh->pair[sw], pair_phase & 1, status, 16))) break;
            ATC_T(3);
            ++pair_phase;
            const float mx = fmaxf(__bfloat162float(mine), __bfloat162float(sh->xmax[half ^ 1][r]));
            // raise the reference only when it is first set or falls too far behind
            const bool raise = mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * sc > ATC_RESCALE_LOG2);
            const bool shrink = raise && m_ref != -INFINITY;          // what this row has accumulated must be rescaled
            const bool rescale = i > 0 && __any_sync(0xffffffffu, shrink);
            const float alpha = shrink ? ex2_approx((m_ref - mx) * sc) : 1.f;
            if (raise) m_ref = mx;
            const float neg = m_ref == -INFINITY ? 0.f : -m_ref * sc;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t w[16];                                           // this half of the row of P, bfloat16 pairs
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const float p0 = ex2_approx(fmaf(s[2 * e], sc, neg)), p1 = ex2_approx(fmaf(s[2 * e + 1], sc, neg));
                sum4[e & 3] += p0 + p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                w[e] = *reinterpret_cast<uint32_t*>(&h2);
            }
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            ATC_T(4);
            // P's buffer and the accumulator belong to the product of the page before until it is done
            if (i > 0) {
                if (!(ok = mbar_wait(&sh->pv_ready, (i - 1) & 1, status, 14))) break;
                tc_fence_after();
            }
            ATC_T(5);
            if (rescale) {       // this warp's rows and half of the columns (rows that keep their reference: factor 1)
#pragma unroll 1
                for (int c = 0; c < HD / 64; ++c) {
                    float ov[32];
                    tc_ld32(tmem_o + lane_base + half * (HD / 2) + c * 32, ov);
#pragma unroll
                    for (int d = 0; d < 32; ++d) ov[d] *= alpha;
                    tc_st32(tmem_o + lane_base + half * (HD / 2) + c * 32, ov);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // P row -> shared memory, 16 bytes (8 keys) at a time, chunk c at position c ^ (row & 7)
            unsigned char* prow = ps + r * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(prow + (((half * 4 + c) ^ (r & 7)) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
            // The page's rows past the sequence's last position may hold anything (an earlier
            // sequence's values): zero them in V, so that 0 * value stays 0.
            if (kt * 64 + 63 > pos_last) {
                if (!(ok = mbar_wait(&sh->v_full[i & 1], (i >> 1) & 1, status, 15))) break;     // V has landed
            }
            if (kt * 64 + 63 > pos_last && half == 0 && r < 64 && kt * 64 + r > pos_last) {
                unsigned char* vrow = vs + (i & 1) * KV_BYTES + r * 128;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<uint4*>(vrow + nb * 64 * 128 + c * 16) = make_uint4(0, 0, 0, 0);
            }
            ATC_T(6);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // P (and the zeros) are for the MMA to read
            tc_fence_before();
            mbar_arrive(&sh->p_ready);
            ATC_T(7);
        }
        if (ok && n_kt > 0) ok = mbar_wait(&sh->pv_ready, (n_kt - 1) & 1, status, 11);
        tc_fence_after();
        // 1 / (sum of both halves): the second half hands its sum over, the first hands the quotient back
        float* xl = reinterpret_cast<float*>(&sh->xmax[0][0]);
        float inv = 0.f;
        if (ok) {
            if (half == 1) xl[r] = l;
            mbar_arrive(&sh->pair[sw]);
            ok = mbar_wait(&sh->pair[sw], pair_phase & 1, status, 16);
            ++pair_phase;
        }
        if (ok) {
            if (half == 0) {
                inv = 1.0f / (l + xl[r]);
                xl[r] = inv;
            }
            mbar_arrive(&sh->pair[sw]);
            ok = mbar_wait(&sh->pair[sw], pair_phase & 1, status, 16);
            ++pair_phase;
        }
        if (!ok) sh->failed = 1;
        if (ok) {
            if (half == 1) inv = xl[r];
            bf16* dst = a.out + (int64_t)(row0 + r) * (a.q_heads * HD) + head * HD + half * (HD / 2);
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                float ov[32];
                tc_ld32(tmem_o + lane_base + half * (HD / 2) + c * 32, ov);      // every lane takes part in the load
                if (r < nrows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        float v8[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v8[e] = ov[d + e] * inv;
                        tc_store8(dst + c * 32 + d, v8);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ATC_TMEM_COLS) : "memory");
    }
}

// ----------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------
template <int HD>
static int launch_attn_tc(const CUtensorMap& map_q, const CUtensorMap& map_kv, const AttnTcArgs& a, const PagedCache& cache,
                          int n_tiles, int* status, cudaStream_t stream) {
    constexpr int NB = HD / 64;
    const size_t smem = (size_t)NB * 128 * 128 + 4 * (size_t)NB * 64 * 128 + 128 * 128 + sizeof(AttnTcShared);
    static OncePerDevice configured;
    if (configured.need()) {
        cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            x0ne_set_error("attention_prefill_tc: cannot set %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured.done();
    }
    x0ne_launch(attention_prefill_tc_kernel<HD>, dim3(a.q_heads, n_tiles), dim3(ATC_THREADS), smem, stream, map_q, map_kv, a,
                cache, status);
    X0NE_LAUNCH_CHECK();
}

// q, out: bfloat16 [q_rows, q_heads * head_dim]; tiles of up to 128 rows (tile tables as for the
// mma.sync prefill kernel).  `status`: one int in device memory, zero before the first call; not
// zero afterwards means a barrier wait ran out and the output is not valid.
X0NE_API int x0ne_attention_prefill_tcgen05(const void* q, void* out, int q_rows, PagedCache cache, const int32_t* tile_seq,
                                            const int32_t* tile_row0, int n_tiles, const int32_t* seq_first_row,
                                            const int32_t* seq_slot, const int32_t* seq_pos0, int q_heads, float scale,
                                            int window, int* status, cudaStream_t stream) {
    X0NE_REQUIRE(cache.page_size == 64, "attention_prefill_tc: pages of %d positions, the kernel takes 64", cache.page_size);
    X0NE_REQUIRE(cache.head_dim == 64 || cache.head_dim == 128, "attention_prefill_tc: head_dim %d (64 or 128)", cache.head_dim);
    X0NE_REQUIRE(q_heads > 0 && cache.kv_heads > 0 && q_heads % cache.kv_heads == 0, "attention_prefill_tc: %d q heads over %d kv heads",
                 q_heads, cache.kv_heads);
    X0NE_REQUIRE(n_tiles >= 0 && n_tiles <= 65535 && window >= 0 && q_rows > 0 && status != nullptr, "attention_prefill_tc: bad sizes");
    X0NE_REQUIRE((int64_t)cache.n_pages * 2 * cache.kv_heads * 64 <= 0x7fffffff, "attention_prefill_tc: the cache has too many rows");
    X0NE_REQUIRE(cache.page_stride == (int64_t)2 * cache.kv_heads * 64 * cache.head_dim, "attention_prefill_tc: pages are not contiguous");
    if (n_tiles == 0) return 0;
    CUtensorMap map_q, map_kv;
    if (int e = x0ne_tc_make_map(&map_q, q, q_rows, (int64_t)q_heads * cache.head_dim, 128)) return e;
    if (int e = x0ne_tc_make_map(&map_kv, cache.base, (int64_t)cache.n_pages * 2 * cache.kv_heads * 64, cache.head_dim, 64)) return e;
    AttnTcArgs a{(bf16*)out, tile_seq, tile_row0, seq_first_row, seq_slot, seq_pos0, q_heads, window, scale * 1.4426950408889634f};
    if (cache.head_dim == 128) return launch_attn_tc<128>(map_q, map_kv, a, cache, n_tiles, status, stream);
    return launch_attn_tc<64>(map_q, map_kv, a, cache, n_tiles, status, stream);
}
