// y[M,N] = x[M,K] W[N,K]^T for bfloat16 with a small M (decode): a weight-streaming kernel.
//
// A decode step multiplies a handful of rows by every weight matrix of the model, so the product
// is bound by reading W once from HBM (the library engine gives these shapes to cublasGemmEx,
// x0ne-core/runtime/src/gpu.rs:1098-1149).  Here W is the A operand of mma.sync m16n8k16: a warp
// takes 16 weight rows and streams them along K with 16-byte asynchronous copies (cp.async.cg,
// which bypasses L1), the M <= 8*MT activation rows are the B operand (copied the same way, from
// L2), and the accumulators are float32.  Because a dot product does not care about the order of its terms, each thread feeds
// the 8 consecutive k values of its 16-byte load to the MMA slots directly (the same permutation on
// both operands), so no shuffle or shared-memory staging is needed.  The 8 warps of a block split K
// in interleaved 32-value chunks and are summed in a fixed order at the end.
//
// Variants: bfloat16 or float32 output (logits), and SwiGLU fused into the epilogue for the packed
// [gate; up] weight (out[m][i] = silu(gate_i . x_m) * (up_i . x_m), in float32, rounded once:
// x0ne-core/kernels/cuda/swiglu.cu:5-11 without the intermediate bfloat16 rounding of gate and up).
// Needs K % 8 == 0; other shapes go to the library product.
#include "common.cuh"

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#define SM_WARPS 8
// Ring depth (chunks per thread) of a variant: the deepest with which two blocks still fit on an
// SM (228 KB, 1 KB of it reserved per block), since what a thread has in flight is what hides the
// memory latency.  Up to 8 rows: 9 chunks, 5 with the SwiGLU epilogue (two weight sets).
constexpr int smallm_depth(int mt, bool swiglu) {
    const int sets = swiglu ? 2 : 1;
    const int slots = sets * 2 + mt;
    const int part = SM_WARPS * sets * mt * 128 * 4;
    const int depth = ((228 * 1024) / 2 - 1024 - part) / (slots * SM_WARPS * 32 * 16);
    return depth < 2 ? 2 : depth;
}
static_assert(smallm_depth(1, false) == 9 && smallm_depth(1, true) == 5 && smallm_depth(2, false) == 6 && smallm_depth(2, true) == 4,
              "ring depths");

// 16 bytes global -> shared, asynchronously; `bytes` = 0 writes zeros instead (out-of-range rows or k).
__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Each thread streams its 16-byte pieces of W through a private ring of DEPTH slots in shared
// memory with cp.async: DEPTH - 1 chunks (2 rows x 16 bytes each, per weight set) are in flight per
// thread whatever the register allocator does, which is what hides the memory latency.  A thread
// reads back only what it copied itself, so no barrier is needed inside the k loop.  A block owns
// the tiles (16 weight rows each) blockIdx.x, blockIdx.x + gridDim.x, ...; the copies run ahead
// across the tile boundary, so the stream does not drain while a tile's partial sums are reduced.
template <int MT, typename OutT, bool SWIGLU, int DEPTH>
__global__ void __launch_bounds__(SM_WARPS * 32) gemm_smallm_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X,
                                                                    OutT* __restrict__ Y, int M, int N, int K, int ldy,
                                                                    int n_tiles) {
    constexpr int SETS = SWIGLU ? 2 : 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int SLOTS = SETS * 2 + MT;     // 16-byte pieces per chunk and thread: weight rows, then activation rows
    uint4* ring = reinterpret_cast<uint4*>(smem_raw);                        // [DEPTH][SLOTS][threads]
    float* part = reinterpret_cast<float*>(ring + DEPTH * SLOTS * SM_WARPS * 32);      // [warps][SETS][MT][128]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int chunks = (K + 31) / 32;
    const int my_chunks = chunks > warp ? (chunks - warp + SM_WARPS - 1) / SM_WARPS : 0;   // chunks warp, warp + 8, ...
    const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    auto slot = [&](int d, int s, int h) -> uint4* { return ring + (d * SLOTS + s * 2 + h) * (SM_WARPS * 32) + tid; };
    auto xslot = [&](int d, int j) -> uint4* { return ring + (d * SLOTS + SETS * 2 + j) * (SM_WARPS * 32) + tid; };

    pdl_launch_dependents();

    // the copies' cursor: tile p_tile of this block, chunk p_chunk of this warp, ring slot p_slot
    int p_tile = 0, p_chunk = 0, p_slot = 0;
    const bool streams = my_chunks > 0 && my_tiles > 0;
    auto issue_w = [&](int tile_j, int i, int d) {
        const int n0 = ((int)blockIdx.x + tile_j * (int)gridDim.x) * 16;
        const int k = (warp + i * SM_WARPS) * 32 + 8 * t;
        const bool kok = k < K;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = n0 + g + 8 * h;
            const bool ok = kok && n < N;
#pragma unroll
            for (int s = 0; s < SETS; ++s)
                cp_async16_zfill(slot(d, s, h), W + (ok ? (int64_t)(s * N + n) * K + k : 0), ok ? 16 : 0);
        }
    };
    auto issue_x = [&](int i, int d) {
        const int k = (warp + i * SM_WARPS) * 32 + 8 * t;
#pragma unroll
        for (int j = 0; j < MT; ++j) {
            const int m = 8 * j + g;
            const bool ok = k < K && m < M;
            cp_async16_zfill(xslot(d, j), X + (ok ? (int64_t)m * K + k : 0), ok ? 16 : 0);
        }
    };
    auto advance = [&]() {
        if (++p_chunk == my_chunks) {
            p_chunk = 0;
            ++p_tile;
        }
        p_slot = p_slot + 1 == DEPTH ? 0 : p_slot + 1;
    };

    // The weights do not depend on the kernel before this one: the first chunks are requested
    // before waiting for it (their copies then all belong to the first commit group, which is
    // harmless: that group is waited for first).
    {
        int jt = 0, ic = 0;
#pragma unroll
        for (int d = 0; d < DEPTH - 1; ++d) {
            if (streams && jt < my_tiles) issue_w(jt, ic, d);
            if (++ic >= my_chunks) { ic = 0; ++jt; }
        }
    }
    pdl_wait();
#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) {
        if (streams && p_tile < my_tiles) issue_x(p_chunk, d);
        cp_commit();
        if (streams) advance();
    }

    int c_slot = 0;
    for (int tile_j = 0; tile_j < my_tiles; ++tile_j) {
        float acc[SETS][MT][4];
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < MT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[s][j][i] = 0.f;
        for (int i = 0; i < my_chunks; ++i) {
            if (p_tile < my_tiles) {
                issue_w(p_tile, p_chunk, p_slot);
                issue_x(p_chunk, p_slot);
            }
            cp_commit();
            advance();
            cp_wait<DEPTH - 1>();
            uint4 b[MT];
#pragma unroll
            for (int j = 0; j < MT; ++j) b[j] = *xslot(c_slot, j);
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                const uint4 a0 = *slot(c_slot, s, 0), a1 = *slot(c_slot, s, 1);
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    mma16816(acc[s][j], a0.x, a1.x, a0.y, a1.y, b[j].x, b[j].y);
                    mma16816(acc[s][j], a0.z, a1.z, a0.w, a1.w, b[j].z, b[j].w);
                }
            }
            c_slot = c_slot + 1 == DEPTH ? 0 : c_slot + 1;
        }
        // partials: part[warp][set][j][row * 8 + col], row = weight row in the tile, col = m in the tile
        const int n0 = ((int)blockIdx.x + tile_j * (int)gridDim.x) * 16;
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                float* p = part + ((warp * SETS + s) * MT + j) * 128;
                p[g * 8 + 2 * t] = acc[s][j][0];
                p[g * 8 + 2 * t + 1] = acc[s][j][1];
                p[(g + 8) * 8 + 2 * t] = acc[s][j][2];
                p[(g + 8) * 8 + 2 * t + 1] = acc[s][j][3];
            }
        __syncthreads();
        for (int e = tid; e < MT * 128; e += SM_WARPS * 32) {
            const int j = e / 128, r = e % 128;
            const int row = r % 16, col = r / 16;      // consecutive threads -> consecutive n
            const int n = n0 + row, m = 8 * j + col;
            float v[SETS];
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < SM_WARPS; ++w) sum += part[((w * SETS + s) * MT + j) * 128 + row * 8 + col];
                v[s] = sum;
            }
            if (n < N && m < M) {
                float out = v[0];
                if (SWIGLU) out = v[0] / (1.0f + expf(-v[0])) * v[SETS - 1];
                Y[(int64_t)m * ldy + n] = from_f32<OutT>(out);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
}

template <int MT, typename OutT, bool SWIGLU>
static int launch_smallm(const bf16* W, const bf16* X, OutT* Y, int M, int N, int K, int ldy, int sms, cudaStream_t stream) {
    constexpr int SETS = SWIGLU ? 2 : 1;
    constexpr int SLOTS = SETS * 2 + MT;
    constexpr int DEPTH = smallm_depth(MT, SWIGLU);
    constexpr int SMEM = DEPTH * SLOTS * SM_WARPS * 32 * 16 + SM_WARPS * SETS * MT * 128 * 4;
    const int n_tiles = (N + 15) / 16;
    static int fit[64];        // per device: blocks of this variant that fit on one SM (0: not asked yet)
    const int dev = OncePerDevice::device();
    int per_sm = dev >= 0 ? fit[dev] : 0;
    if (per_sm == 0) {
        auto kernel = gemm_smallm_kernel<MT, OutT, SWIGLU, DEPTH>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) {
            x0ne_set_error("gemm_smallm: cannot set %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
            return (int)e;
        }
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, SM_WARPS * 32, SMEM) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
        if (dev >= 0) fit[dev] = n;
    }
    // Every block gets the same number of tiles (but for the remainder), and no more blocks are
    // launched than are resident at once: the blocks then end together.
    const int resident = sms * per_sm;
    const int tiles_per_block = (n_tiles + resident - 1) / resident;
    const int grid = (n_tiles + tiles_per_block - 1) / tiles_per_block;
    x0ne_launch(gemm_smallm_kernel<MT, OutT, SWIGLU, DEPTH>, dim3(grid), dim3(SM_WARPS * 32), SMEM, stream, W, X, Y, M, N, K, ldy, n_tiles);
    X0NE_LAUNCH_CHECK();
}

// out_kind: 0 = bfloat16, 1 = float32, 2 = bfloat16 with SwiGLU over the packed [gate; up] weight
// (W then has 2*N rows and y has N columns).
X0NE_API int x0ne_gemm_bf16_smallm(const void* W, const void* X, void* Y, int M, int N, int K, int ldy, int out_kind,
                                   int sms, cudaStream_t stream) {
    X0NE_REQUIRE(M >= 0 && M <= 32 && N > 0 && K > 0, "gemm_smallm: M %d (at most 32) N %d K %d", M, N, K);
    X0NE_REQUIRE(K % 8 == 0, "gemm_smallm: K %d is not a multiple of 8", K);
    X0NE_REQUIRE(ldy >= N && sms > 0 && out_kind >= 0 && out_kind <= 2, "gemm_smallm: ldy %d N %d kind %d", ldy, N, out_kind);
    X0NE_REQUIRE((((uintptr_t)W | (uintptr_t)X) & 15) == 0, "gemm_smallm: operands are not 16-byte aligned");
    if (M == 0) return 0;
    const bf16* w = (const bf16*)W;
    const bf16* x = (const bf16*)X;
    const int mt = (M + 7) / 8;
#define X0NE_SMALLM(MT)                                                                                        \
    if (out_kind == 0) return launch_smallm<MT, bf16, false>(w, x, (bf16*)Y, M, N, K, ldy, sms, stream);       \
    if (out_kind == 1) return launch_smallm<MT, float, false>(w, x, (float*)Y, M, N, K, ldy, sms, stream);     \
    return launch_smallm<MT, bf16, true>(w, x, (bf16*)Y, M, N, K, ldy, sms, stream);
    if (mt == 1) { X0NE_SMALLM(1) }
    if (mt == 2) { X0NE_SMALLM(2) }
    { X0NE_SMALLM(4) }
#undef X0NE_SMALLM
}
