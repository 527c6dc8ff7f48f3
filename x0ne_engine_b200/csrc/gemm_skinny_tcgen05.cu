// y[M,N] = x[M,K] W[N,K]^T for bfloat16 with 9 to 64 rows (decode at batches the weight-streaming
// mma.sync kernel does not take, short prompts): the product is bound by reading W once, so W is
// the big operand of the MMA and the work is cut so that every SM streams an equal share.  The
// library engine gives these shapes to cublasGemmEx (x0ne-core/runtime/src/gpu.rs:1098-1149).
//
//   * A tile is 128 rows of W (tcgen05.mma M = 128) against all rows of x (N = M rounded up to 16,
//     at most 64), K = 16 per instruction; the accumulator [128 weight rows][rows of x] lives in
//     tensor memory.
//   * K is cut into `slices` equal parts, one block each, so that tiles x slices fill the GPU with
//     two blocks per SM.  The blocks of a tile are one thread-block cluster: each leaves its
//     partial sums in its shared memory, and after a cluster barrier every block adds the partial
//     sums of a share of the rows in the order of the slices (through distributed shared memory:
//     no scratch in global memory, no atomics, the same bits every time) and writes them.
//   * Inside a block: warp 4 copies (TMA, 128-byte swizzle, 4 stages of 16 KB of W + 8 KB of x;
//     the W copies of the first stages are issued before the kernel waits for its predecessor, the
//     x copies after), warp 5 issues the MMAs and commits to the stages' "empty" barriers, warps
//     0-3 read the accumulator when the last MMA is done.
//   * With SwiGLU a tile is 64 gate rows and the 64 up rows that pair with them (weight [gate; up]
//     of 2 N rows), and the block that adds a row up writes silu(gate) * up
//     (x0ne-core/kernels/cuda/swiglu.cu:5-11 without the intermediate bfloat16 rounding).
//
// Every barrier wait is bounded (about a second); when one runs out the block sets its bit in
// `status`, still joins the cluster barriers and frees its tensor memory, and writes nothing.
#include <stdlib.h>

#include "tcgen05.cuh"

#define SK_STAGES 4
#define SK_BK 64
#define SK_XROWS 64
#define SK_THREADS 192
#define SK_TMEM_COLS 64
#define SK_MAX_SLICES 8

struct SkShared {
    uint64_t full[SK_STAGES];
    uint64_t empty[SK_STAGES];
    uint64_t accum;
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ uint32_t sk_cluster_addr(const void* local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(tc_smem(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ float sk_ld_cluster(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 sk_ld_cluster4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sk_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// grid: (slices, tiles); with slices > 1 the blocks of one tile are a cluster along x.
template <bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(SK_THREADS, 2) gemm_skinny_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                       const __grid_constant__ CUtensorMap map_w,
                                                                       OutT* __restrict__ Y, int M, int N, int K, int ldy,
                                                                       int mma_n, int* status) {
    extern __shared__ unsigned char sk_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sk_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = 128 * 128, B_BYTES = SK_XROWS * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    SkShared* sh = reinterpret_cast<SkShared*>(base + SK_STAGES * STAGE_BYTES);
    float* part = reinterpret_cast<float*>(base);      // [rows of x][128]: this block's sums, once the stages are done with
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int slices = gridDim.x, slice = blockIdx.x, tile = blockIdx.y;
    constexpr int COLS = SWIGLU ? 64 : 128;             // columns of y per tile
    const int n0 = tile * COLS;
    const int k_blocks = (K + SK_BK - 1) / SK_BK;
    const int kb_lo = (int)(((int64_t)k_blocks * slice) / slices), kb_hi = (int)(((int64_t)k_blocks * (slice + 1)) / slices);
    const int n_kb = kb_hi - kb_lo;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->accum, 1);
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)),
                     "r"(SK_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 4) {
        // ---- copies.  All lanes run the loop; one elected lane issues, and the warp comes together
        // again before anyone waits.
        uint32_t leader = 0;
        asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
        auto load_w = [&](int i) {
            const int s = i % SK_STAGES;
            unsigned char* a = base + s * STAGE_BYTES;
            if (leader) {
                mbar_expect_tx(&sh->full[s], STAGE_BYTES);
                if (SWIGLU) {
                    tma_load_2d(a, &map_w, (kb_lo + i) * SK_BK, n0, &sh->full[s]);                  // 64 gate rows
                    tma_load_2d(a + 64 * 128, &map_w, (kb_lo + i) * SK_BK, N + n0, &sh->full[s]);   // 64 up rows
                } else {
                    tma_load_2d(a, &map_w, (kb_lo + i) * SK_BK, n0, &sh->full[s]);
                }
            }
            __syncwarp();
        };
        auto load_x = [&](int i) {
            const int s = i % SK_STAGES;
            if (leader) tma_load_2d(base + s * STAGE_BYTES + A_BYTES, &map_x, (kb_lo + i) * SK_BK, 0, &sh->full[s]);
            __syncwarp();
        };
        const int ahead = n_kb < SK_STAGES ? n_kb : SK_STAGES;
        for (int i = 0; i < ahead; ++i) load_w(i);      // the weights do not depend on the kernel before this one
        pdl_wait();
        for (int i = 0; i < ahead; ++i) load_x(i);
        bool ok = true;
        for (int i = SK_STAGES; i < n_kb && ok; ++i) {
            ok = __all_sync(0xffffffffu, mbar_wait(&sh->empty[i % SK_STAGES], ((i / SK_STAGES) - 1) & 1, status, 1));
            if (!ok) break;
            load_w(i);
            load_x(i);
        }
        if (!ok) sh->failed = 1;
    } else if (warp == 5) {
        // ---- products
        uint32_t leader = 0;
        asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)mma_n >> 3) << 17) | ((128u >> 4) << 24);
        bool ok = true;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % SK_STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&sh->full[s], (i / SK_STAGES) & 1, status, 2));
            if (!ok) break;
            tc_fence_after();
            if (leader) {
                const uint32_t a = tc_smem(base + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                for (int k = 0; k < SK_BK / 16; ++k)
                    tc_mma(tmem, tc_desc(a + k * 32), tc_desc(b + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(&sh->empty[s]);
                if (i == n_kb - 1) tc_commit(&sh->accum);
            }
            __syncwarp();
        }
        if (!ok) sh->failed = 1;
    } else {
        // ---- the accumulator: lane r of tensor memory = weight row r of the tile; column m = row m of x
        bool ok = n_kb > 0 ? mbar_wait(&sh->accum, 0, status, 3) : true;
        tc_fence_after();
        if (!ok) sh->failed = 1;
        const int r = warp * 32 + lane;
        const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < SK_TMEM_COLS / 32; ++c) {
            float v[32];
            if (n_kb > 0 && ok) {
                tc_ld32(trow + c * 32, v);      // columns past the rows of x hold nothing; they are not used
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (c * 32 + i < M) part[(c * 32 + i) * 128 + r] = v[i];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (slices > 1) sk_cluster_sync();
    // A block's failure is local; the others cannot see it, so every block writes its share unless
    // it failed itself (the status word tells the host that the result is not valid).
    if (!sh->failed) {
        // This block's share: groups of four consecutive columns of the rows slice, slice + slices, ...
        // All loads of a group are issued before the first sum (they are independent), then added
        // in the order of the slices.
        constexpr int GROUPS = COLS / 4;
        const int my_rows = M > slice ? (M - slice + slices - 1) / slices : 0;
        uint32_t peer[SK_MAX_SLICES];
#pragma unroll
        for (int s = 0; s < SK_MAX_SLICES; ++s) peer[s] = sk_cluster_addr(part, (uint32_t)(s < slices ? s : 0));
        for (int e = threadIdx.x; e < my_rows * GROUPS; e += SK_THREADS) {
            const int m = slice + (e / GROUPS) * slices, c = (e % GROUPS) * 4;
            const uint32_t off = (uint32_t)(m * 128 + c) * 4;
            float4 g[SK_MAX_SLICES], u[SK_MAX_SLICES];
#pragma unroll
            for (int s = 0; s < SK_MAX_SLICES; ++s) {
                if (s < slices) {
                    g[s] = sk_ld_cluster4(peer[s] + off);
                    if (SWIGLU) u[s] = sk_ld_cluster4(peer[s] + off + 64 * 4);
                }
            }
            float4 gs = make_float4(0.f, 0.f, 0.f, 0.f), us = gs;
#pragma unroll
            for (int s = 0; s < SK_MAX_SLICES; ++s) {
                if (s < slices) {
                    gs.x += g[s].x; gs.y += g[s].y; gs.z += g[s].z; gs.w += g[s].w;
                    if (SWIGLU) { us.x += u[s].x; us.y += u[s].y; us.z += u[s].z; us.w += u[s].w; }
                }
            }
            float o4[4] = {gs.x, gs.y, gs.z, gs.w};
            if (SWIGLU) {
                const float u4[4] = {us.x, us.y, us.z, us.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) o4[i] = o4[i] / (1.0f + expf(-o4[i])) * u4[i];
            }
            const int n = n0 + c;
            OutT* dst = Y + (int64_t)m * ldy + n;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n + i < N) dst[i] = from_f32<OutT>(o4[i]);
        }
    }
    if (slices > 1) sk_cluster_sync();      // nobody leaves while its sums may still be read
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(SK_TMEM_COLS) : "memory");
    }
}

// ----------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------
int x0ne_tc_make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int box_rows);

template <bool SWIGLU, typename OutT>
static int launch_skinny(const void* W, const void* X, int x_rows, OutT* Y, int M, int N, int K, int ldy, int* status,
                         cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    // The map covers the rows x really has (up to the tile's 64): rows past M then come from memory
    // instead of being filled with zeros, which is faster when M is below 16 (a third, measured) and
    // harmless, since the columns of the accumulator they produce are never read.
    if (int e = x0ne_tc_make_map(&map_x, X, x_rows < SK_XROWS ? x_rows : SK_XROWS, K, SK_XROWS)) return e;
    if (int e = x0ne_tc_make_map(&map_w, W, SWIGLU ? 2 * (int64_t)N : N, K, SWIGLU ? 64 : 128)) return e;
    const size_t smem = (size_t)SK_STAGES * (128 * 128 + SK_XROWS * 128) + sizeof(SkShared) + 1024;
    static OncePerDevice configured;
    if (configured.need()) {
        cudaFuncSetAttribute(gemm_skinny_tc_kernel<SWIGLU, OutT>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_tc_kernel<SWIGLU, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            x0ne_set_error("gemm_skinny_tc: cannot set %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured.done();
    }
    constexpr int COLS = SWIGLU ? 64 : 128;
    const int tiles = (N + COLS - 1) / COLS;
    X0NE_REQUIRE(tiles <= 65535, "gemm_skinny_tc: %d tiles (limit 65535)", tiles);
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 1;
    // As many slices of K as keep tiles x slices within the blocks resident at once (two per SM,
    // less an eighth: clusters do not pack the GPCs completely, and a launch that does not fit at
    // once costs a second wave: 48 tiles x 6 slices took 16.8 us, x 4 slices 11.8 us), at least
    // four 64-wide k blocks each, at most a portable cluster.
    const int k_blocks = (K + SK_BK - 1) / SK_BK;
    int slices = (2 * sms - 2 * sms / 8) / tiles;
    if (slices > SK_MAX_SLICES) slices = SK_MAX_SLICES;
    if (slices > k_blocks / 4) slices = k_blocks / 4;
    if (slices < 1) slices = 1;
    if (const char* e = getenv("X0NE_SK_SLICES")) {      // experiments
        const int v = atoi(e);
        if (v >= 1 && v <= SK_MAX_SLICES && v <= k_blocks) slices = v;
    }
    const int mma_n = (M + 15) / 16 * 16;
    if (slices > 1)
        x0ne_launch_clusters(gemm_skinny_tc_kernel<SWIGLU, OutT>, dim3(slices, tiles), dim3(SK_THREADS), slices, smem, stream, map_x,
                             map_w, Y, M, N, K, ldy, mma_n, status);
    else
        x0ne_launch(gemm_skinny_tc_kernel<SWIGLU, OutT>, dim3(1, tiles), dim3(SK_THREADS), smem, stream, map_x, map_w, Y, M, N, K,
                    ldy, mma_n, status);
    X0NE_LAUNCH_CHECK();
}

// out_kind: 0 = bfloat16, 1 = float32, 2 = bfloat16 with SwiGLU over the packed [gate; up] weight
// (W then has 2*N rows and y has N columns).  `status` as for the other tcgen05 kernels.
// `x_rows`: rows allocated behind X (at least M).
X0NE_API int x0ne_gemm_bf16_skinny_tcgen05(const void* W, const void* X, int x_rows, void* Y, int M, int N, int K, int ldy,
                                           int out_kind, int* status, cudaStream_t stream) {
    X0NE_REQUIRE(M >= 0 && M <= 64 && N > 0 && K > 0 && x_rows >= M, "gemm_skinny_tc: M %d (at most 64, x has %d rows) N %d K %d", M, x_rows, N, K);
    X0NE_REQUIRE(K % 8 == 0, "gemm_skinny_tc: K %d is not a multiple of 8 (rows must be 16-byte aligned for TMA)", K);
    X0NE_REQUIRE(ldy >= N && out_kind >= 0 && out_kind <= 2 && status != nullptr, "gemm_skinny_tc: ldy %d N %d kind %d", ldy, N, out_kind);
    X0NE_REQUIRE((((uintptr_t)W | (uintptr_t)X) & 15) == 0, "gemm_skinny_tc: operands are not 16-byte aligned");
    if (M == 0) return 0;
    if (out_kind == 0) return launch_skinny<false, bf16>(W, X, x_rows, (bf16*)Y, M, N, K, ldy, status, stream);
    if (out_kind == 1) return launch_skinny<false, float>(W, X, x_rows, (float*)Y, M, N, K, ldy, status, stream);
    return launch_skinny<true, bf16>(W, X, x_rows, (bf16*)Y, M, N, K, ldy, status, stream);
}
