// y[M,N] = x[M,K] W[N,K]^T for bfloat16 on the 5th-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands brought to shared memory by TMA, an mbarrier pipeline
// between a copy thread, an MMA thread and four epilogue warps.  For passes with many rows
// (prefill); the library engine gives these products to cublasGemmEx
// (x0ne-core/runtime/src/gpu.rs:1098-1149).
//
// A block computes 128 x 256 tiles of y, one after another:
//   * warp 0, one thread: for every 64-wide slice of K, waits until the stage is free, then issues
//     two TMA tile loads (x: 128 rows x 128 bytes, W: 256 rows x 128 bytes, 128-byte swizzle) that
//     complete on the stage's "full" barrier.  Rows or k values past the matrices read as zeros.
//   * warp 1, one thread: waits for "full", issues four tcgen05.mma (M 128, N 256, K 16) whose
//     shared-memory descriptors step 32 bytes through the swizzled slice, then tcgen05.commit to the
//     stage's "empty" barrier (the stage is free when those MMAs are done); after the last slice,
//     commits to the "accumulator ready" barrier.
//   * warps 2-5: wait for it, read their 32 rows of the accumulator with tcgen05.ld, convert, store.
// With SwiGLU the W tile is 128 gate rows and the 128 up rows that pair with them, the two halves
// accumulate side by side, and the epilogue writes silu(gate) * up (x0ne-core/kernels/cuda/
// swiglu.cu:5-11 without the intermediate bfloat16 rounding).
//
// Every block fetches its own operands.  Every barrier wait is bounded (about a second); when one runs out the
// kernel records where in `status`, skips the rest, still frees its tensor memory, and returns.
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_STAGES 4
#define TC_THREADS 192
#define TC_TMEM_COLS 512

struct TcShared {
    uint64_t full[TC_STAGES];
    uint64_t empty[TC_STAGES];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint32_t tmem_base;
    int failed;
};

// SWIGLU: W is the packed [gate; up] weight of 2 * N rows; a tile's W operand is gate rows
// n0 .. n0 + 127 and up rows N + n0 .. N + n0 + 127, and y has N columns.
//
// Blocks are persistent: block b takes tiles b, b + gridDim.x, ...; consecutive tile numbers walk
// down the rows of y first, so the blocks running at one time share a few W tiles (read once from
// HBM, then from L2) and all of x stays in L2.  The accumulator is double-buffered in tensor memory
// (2 x 256 columns): the epilogue of one tile runs while the MMAs of the next are issued.
template <bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                                                             const __grid_constant__ CUtensorMap map_w, OutT* __restrict__ Y,
                                                             int M, int N, int K, int ldy, int m_tiles, int n_tiles,
                                                             int* status) {
    extern __shared__ unsigned char tc_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = TC_BM * 128, B_BYTES = 256 * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    TcShared* sh = reinterpret_cast<TcShared*>(base + TC_STAGES * STAGE_BYTES);
    constexpr int BN = SWIGLU ? 128 : 256;      // columns of y per tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int tiles = m_tiles * n_tiles;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh->accum_full[b], 1);
            mbar_init(&sh->accum_empty[b], 128);
        }
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)),
                     "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();      // x was written by the kernel before this one
            int it = 0;      // k-slices issued so far, over all tiles
            for (int tile = blockIdx.x; tile < tiles && !sh->failed; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TC_STAGES;
                    if (it >= TC_STAGES && !mbar_wait(&sh->empty[s], ((it / TC_STAGES) - 1) & 1, status, 1)) {
                        sh->failed = 1;
                        break;
                    }
                    unsigned char* a = base + s * STAGE_BYTES;
                    unsigned char* b = a + A_BYTES;
                    mbar_expect_tx(&sh->full[s], STAGE_BYTES);
                    tma_load_2d(a, &map_x, kb * TC_BK, m0, &sh->full[s]);
                    if (SWIGLU) {
                        tma_load_2d(b, &map_w, kb * TC_BK, n0, &sh->full[s]);
                        tma_load_2d(b + 128 * 128, &map_w, kb * TC_BK, N + n0, &sh->full[s]);
                    } else {
                        tma_load_2d(b, &map_w, kb * TC_BK, n0, &sh->full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, M = 128
            const uint32_t idesc_n = SWIGLU ? 128u : 256u;
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((idesc_n >> 3) << 17) | ((128u >> 4) << 24);
            int it = 0, t = 0;
            for (int tile = blockIdx.x; tile < tiles && !sh->failed; tile += gridDim.x, ++t) {
                const int ab = t & 1;
                const uint32_t acc_tmem = tmem + ab * 256;
                // the epilogue must have drained this accumulator (two tiles ago)
                if (t >= 2 && !mbar_wait(&sh->accum_empty[ab], ((t >> 1) - 1) & 1, status, 4)) {
                    sh->failed = 1;
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TC_STAGES;
                    if (!mbar_wait(&sh->full[s], (it / TC_STAGES) & 1, status, 2)) {
                        sh->failed = 1;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a = tc_smem(base + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        if (SWIGLU) {
                            tc_mma(acc_tmem, tc_desc(a + k * 32), tc_desc(b + k * 32), idesc, acc);
                            tc_mma(acc_tmem + 128, tc_desc(a + k * 32), tc_desc(b + 128 * 128 + k * 32), idesc, acc);
                        } else {
                            tc_mma(acc_tmem, tc_desc(a + k * 32), tc_desc(b + k * 32), idesc, acc);
                        }
                    }
                    tc_commit(&sh->empty[s]);      // arrives when the MMAs above have read the stage
                }
                tc_commit(&sh->accum_full[ab]);    // arrives when every MMA of this tile is done
            }
        }
    } else {
        // epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. 32 (w % 4) + 31 = rows of the tile
        const int quarter = warp & 3;
        int t = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
            const int ab = t & 1;
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
            const int m = m0 + quarter * 32 + lane;
            if (!mbar_wait(&sh->accum_full[ab], (t >> 1) & 1, status, 3) || sh->failed) {
                sh->failed = 1;
                break;
            }
            tc_fence_after();
            const uint32_t trow = tmem + ab * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < 128 / 32 * (SWIGLU ? 1 : 2); ++c) {
                float v[32];
                tc_ld32(trow + c * 32, v);
                if (SWIGLU) {
                    float u[32];
                    tc_ld32(trow + 128 + c * 32, u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.0f + expf(-v[i])) * u[i];
                }
                const int n = n0 + c * 32;
                if (m < M) {
                    OutT* dst = Y + (int64_t)m * ldy + n;
                    if (n + 32 <= N && (((uintptr_t)dst) & 31) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) tc_store8(dst + i, v + i);
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (n + i < N) dst[i] = from_f32<OutT>(v[i]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&sh->accum_empty[ab]);     // this thread is done with the accumulator
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ----------------------------------------------------------------------------------------
// The same product with pairs of blocks (a cluster of two, tcgen05 cta_group::2): a pair computes a
// 256 x 256 tile.  Each block of the pair brings 128 rows of x and 128 rows of W per k-slice into
// its own shared memory and keeps its 128 rows of the accumulator in its own tensor memory; one
// thread of the pair's first block issues the MMAs (M 256, N 256, K 16), which read both blocks'
// shared memory.  Per flop, half as many bytes cross from L2 to shared memory as with single
// blocks, and a stage is 32 KB, so six stages fit.
//   * "full" barriers live in the first block and count the bytes of both blocks' copies (the
//     second block's copies name the first block's barrier; each block fetches its own operands);
//   * tcgen05.commit arrives on the "empty" and "accumulator ready" barriers of both blocks;
//   * the epilogue threads of both blocks arrive on the first block's "accumulator drained" barrier.
// With SwiGLU the first block's W rows are the gate rows and the second block's the up rows, so the
// accumulator's columns 0-127 are gate and 128-255 up, in both blocks.
// ----------------------------------------------------------------------------------------
#define TC2_STAGES 6

struct Tc2Shared {
    uint64_t full[TC2_STAGES];
    uint64_t empty[TC2_STAGES];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint32_t tmem_base;
    int failed;
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
// The address of `local` (a shared-memory address of this block) in block `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(tc_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both blocks of the pair
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(tc_smem(bar)), "h"((uint16_t)3) : "memory");
}

template <bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  OutT* __restrict__ Y, int M, int N, int K, int ldy,
                                                                  int m_tiles, int n_tiles, int* status) {
    extern __shared__ unsigned char tc_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = 128 * 128, B_BYTES = 128 * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    Tc2Shared* sh = reinterpret_cast<Tc2Shared*>(base + TC2_STAGES * STAGE_BYTES);
    constexpr int BN = SWIGLU ? 128 : 256;      // columns of y per tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int tiles = m_tiles * n_tiles;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < TC2_STAGES; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh->accum_full[b], 1);
            mbar_init(&sh->accum_empty[b], 256);     // the epilogue threads of both blocks
        }
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)),
                     "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();          // both blocks' barriers are initialised before either block uses the other's
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            int it = 0;
            for (int tile = pair; tile < tiles && !sh->failed; tile += pairs) {
                const int m0 = (tile % m_tiles) * 256 + 128 * (int)rank;
                const int n_row = SWIGLU ? (int)rank * N + (tile / m_tiles) * BN : (tile / m_tiles) * BN + 128 * (int)rank;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TC2_STAGES;
                    if (it >= TC2_STAGES && !mbar_wait(&sh->empty[s], ((it / TC2_STAGES) - 1) & 1, status, 1)) {
                        sh->failed = 1;
                        break;
                    }
                    unsigned char* a = base + s * STAGE_BYTES;
                    unsigned char* b = a + A_BYTES;
                    // the first block's barrier counts the bytes of both blocks
                    const uint32_t bar0 = cluster_addr(tc_smem(&sh->full[s]), 0);
                    if (rank == 0) mbar_expect_tx(&sh->full[s], 2 * STAGE_BYTES);
                    tma_load_2d_pair(a, &map_x, kb * TC_BK, m0, bar0);
                    tma_load_2d_pair(b, &map_w, kb * TC_BK, n_row, bar0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, M = 256 over the pair, N = 256
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
            int it = 0, t = 0;
            for (int tile = pair; tile < tiles && !sh->failed; tile += pairs, ++t) {
                const int ab = t & 1;
                const uint32_t acc_tmem = tmem + ab * 256;
                if (t >= 2 && !mbar_wait(&sh->accum_empty[ab], ((t >> 1) - 1) & 1, status, 4)) {
                    sh->failed = 1;
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TC2_STAGES;
                    if (!mbar_wait(&sh->full[s], (it / TC2_STAGES) & 1, status, 2)) {
                        sh->failed = 1;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a = tc_smem(base + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma_pair(acc_tmem, tc_desc(a + k * 32), tc_desc(b + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(&sh->empty[s]);
                }
                tc_commit_pair(&sh->accum_full[ab]);
            }
        }
    } else {
        const int quarter = warp & 3;
        int t = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++t) {
            const int ab = t & 1;
            const int m0 = (tile % m_tiles) * 256 + 128 * (int)rank, n0 = (tile / m_tiles) * BN;
            const int m = m0 + quarter * 32 + lane;
            if (!mbar_wait(&sh->accum_full[ab], (t >> 1) & 1, status, 3) || sh->failed) {
                sh->failed = 1;
                break;
            }
            tc_fence_after();
            const uint32_t trow = tmem + ab * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < 128 / 32 * (SWIGLU ? 1 : 2); ++c) {
                float v[32];
                tc_ld32(trow + c * 32, v);
                if (SWIGLU) {
                    float u[32];
                    tc_ld32(trow + 128 + c * 32, u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.0f + expf(-v[i])) * u[i];
                }
                const int n = n0 + c * 32;
                if (m < M) {
                    OutT* dst = Y + (int64_t)m * ldy + n;
                    if (n + 32 <= N && (((uintptr_t)dst) & 31) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) tc_store8(dst + i, v + i);
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (n + i < N) dst[i] = from_f32<OutT>(v[i]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(cluster_addr(tc_smem(&sh->accum_empty[ab]), 0));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();          // neither block leaves while the other may still touch its memory or barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ----------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, cols] row-major bfloat16 matrix, boxes of box_rows x 64 values, 128-byte swizzle, zeros outside.
int x0ne_tc_make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    X0NE_REQUIRE(fn != nullptr, "gemm_tc: the driver has no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    X0NE_REQUIRE(r == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <bool SWIGLU, typename OutT>
static int launch_tc(const void* W, const void* X, OutT* Y, int M, int N, int K, int ldy, int* status, cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    if (int e = x0ne_tc_make_map(&map_x, X, M, K, TC_BM)) return e;
    if (int e = x0ne_tc_make_map(&map_w, W, SWIGLU ? 2 * (int64_t)N : N, K, SWIGLU ? 128 : 256)) return e;
    const size_t smem = (size_t)TC_STAGES * (TC_BM * 128 + 256 * 128) + sizeof(TcShared) + 1024;
    static OncePerDevice configured;
    if (configured.need()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<SWIGLU, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            x0ne_set_error("gemm_tc: cannot set %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured.done();
    }
    constexpr int BN = SWIGLU ? 128 : 256;
    const int n_tiles = (N + BN - 1) / BN, m_tiles = (M + TC_BM - 1) / TC_BM;
    X0NE_REQUIRE((int64_t)n_tiles * m_tiles <= 0x7fffffff, "gemm_tc: too many tiles");
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 1;
    const int tiles = n_tiles * m_tiles;
    const int grid = tiles < sms ? tiles : sms;      // one persistent block per SM (shared memory allows no more)
    x0ne_launch(gemm_tc_kernel<SWIGLU, OutT>, dim3(grid), dim3(TC_THREADS), smem, stream, map_x, map_w, Y, M, N, K, ldy, m_tiles,
                n_tiles, status);
    X0NE_LAUNCH_CHECK();
}

template <bool SWIGLU, typename OutT>
static int launch_tc_pair(const void* W, const void* X, OutT* Y, int M, int N, int K, int ldy, int* status, cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    if (int e = x0ne_tc_make_map(&map_x, X, M, K, 128)) return e;
    if (int e = x0ne_tc_make_map(&map_w, W, SWIGLU ? 2 * (int64_t)N : N, K, 128)) return e;
    const size_t smem = (size_t)TC2_STAGES * (128 * 128 * 2) + sizeof(Tc2Shared) + 1024;
    static OncePerDevice configured;
    if (configured.need()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<SWIGLU, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            x0ne_set_error("gemm_tc_pair: cannot set %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured.done();
    }
    constexpr int BN = SWIGLU ? 128 : 256;
    const int n_tiles = (N + BN - 1) / BN, m_tiles = (M + 255) / 256;
    X0NE_REQUIRE((int64_t)n_tiles * m_tiles <= 0x7fffffff, "gemm_tc_pair: too many tiles");
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = n_tiles * m_tiles;
    int pairs = sms / 2 > 0 ? sms / 2 : 1;
    if (tiles < pairs) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<SWIGLU, OutT>, map_x, map_w, Y, M, N, K, ldy, m_tiles, n_tiles, status);
    X0NE_LAUNCH_CHECK();
}

// out_kind: 0 = bfloat16, 1 = float32, 2 = bfloat16 with SwiGLU over the packed [gate; up] weight
// (W then has 2*N rows and y has N columns).  `status` is one int in device memory, zero before the
// first call; a non-zero value afterwards says a barrier wait ran out (1 copy, 2 MMA, 3 epilogue)
// and the output is not valid.
// `pair` = 1 uses pairs of blocks (256 x 256 tiles), 0 single blocks (128 x 256 tiles).
X0NE_API int x0ne_gemm_bf16_tcgen05(const void* W, const void* X, void* Y, int M, int N, int K, int ldy, int out_kind,
                                    int pair, int* status, cudaStream_t stream) {
    X0NE_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: M %d N %d K %d", M, N, K);
    X0NE_REQUIRE(K % 8 == 0, "gemm_tc: K %d is not a multiple of 8 (rows must be 16-byte aligned)", K);
    X0NE_REQUIRE(ldy >= N && out_kind >= 0 && out_kind <= 2 && status != nullptr, "gemm_tc: ldy %d N %d kind %d", ldy, N, out_kind);
    X0NE_REQUIRE((((uintptr_t)W | (uintptr_t)X) & 15) == 0, "gemm_tc: operands are not 16-byte aligned");
    if (pair) {
        if (out_kind == 0) return launch_tc_pair<false, bf16>(W, X, (bf16*)Y, M, N, K, ldy, status, stream);
        if (out_kind == 1) return launch_tc_pair<false, float>(W, X, (float*)Y, M, N, K, ldy, status, stream);
        return launch_tc_pair<true, bf16>(W, X, (bf16*)Y, M, N, K, ldy, status, stream);
    }
    if (out_kind == 0) return launch_tc<false, bf16>(W, X, (bf16*)Y, M, N, K, ldy, status, stream);
    if (out_kind == 1) return launch_tc<false, float>(W, X, (float*)Y, M, N, K, ldy, status, stream);
    return launch_tc<true, bf16>(W, X, (bf16*)Y, M, N, K, ldy, status, stream);
}
