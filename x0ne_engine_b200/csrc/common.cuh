// Shared device and host helpers of every kernel file.
//
// Conventions (the same as x0ne-core/kernels/cuda/x0ne_kernels.h:1-3 states for its
// kernels): C linkage for every entry point, row-major tensors, 32-bit accumulation,
// token ids / positions / slots read from device memory, and every index checked without
// trapping: an id outside the vocabulary gives a zero row, a position with no page writes
// nothing.  Reductions run in a fixed order, so a row's result does not depend on what else
// is in the launch (x0ne-core/kernels/cuda/common.cuh:1,24-44).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define X0NE_API extern "C" __attribute__((visibility("default")))

// dtype tags of the C interface
#define X0NE_F32 0
#define X0NE_BF16 1

// Error codes of the C interface (0 = ok; positive values below 10000 are cudaError_t).
#define X0NE_ERR_ARG 10001

void x0ne_set_error(const char* fmt, ...);

#define X0NE_REQUIRE(cond, ...)            \
    do {                                   \
        if (!(cond)) {                     \
            x0ne_set_error(__VA_ARGS__);   \
            return X0NE_ERR_ARG;           \
        }                                  \
    } while (0)

#define X0NE_LAUNCH_CHECK()                                          \
    do {                                                             \
        cudaError_t e_ = cudaGetLastError();                         \
        if (e_ != cudaSuccess) {                                     \
            x0ne_set_error("%s:%d: %s", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return (int)e_;                                          \
        }                                                            \
        return 0;                                                    \
    } while (0)

// Programmatic dependent launch.  Every kernel of this library is launched so that it may start
// while the kernel before it in the stream is still running (its blocks are scheduled and run
// their prologue early); `pdl_wait` then blocks until that kernel has finished and its writes
// are visible.  A kernel calls `pdl_launch_dependents` at once, to let its own successor start
// early in turn, and `pdl_wait` before it touches anything an earlier kernel may have written,
// and before its own first write.  Only reads of weights may come before the wait.
// Set X0NE_PDL=0 in the environment to launch everything fully serialized.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
    pdl_launch_dependents();
    pdl_wait();
}

bool x0ne_pdl_enabled();

// Set-up that the runtime keeps per device (a kernel's shared-memory attribute, occupancy numbers)
// is done once per device, by the first call with that device current: `need()` says whether it
// is still to do, `done()` records it.  Two host threads making the first call on a device at the
// same moment would both do it, which is harmless (the same values are set twice).
struct OncePerDevice {
    unsigned char set[64] = {};
    static int device() {
        int d = 0;
        return cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 64 ? d : -1;
    }
    bool need() const {
        const int d = device();
        return d < 0 || !set[d];
    }
    void done() {
        const int d = device();
        if (d >= 0) set[d] = 1;
    }
};

template <typename... KArgs, typename... Args>
static inline cudaError_t x0ne_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = x0ne_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid cut into clusters of `cluster_x` consecutive blocks along x (grid.x must be
// a multiple of it): blocks of a cluster run at the same time and can read each other's shared memory.
template <typename... KArgs, typename... Args>
static inline cudaError_t x0ne_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, int cluster_x, size_t smem,
                                               cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = x0ne_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// Reductions.  One butterfly over the lanes of a warp and one two-level form over a block, both
// with the combining operation as a parameter; every lane / thread gets the result, and the order
// in which values meet depends on lane and warp numbers only, never on the data or on what else
// runs (the fixed-order rule of x0ne-core/kernels/cuda/common.cuh:1).
struct OpSum {
    template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return a + b; }
};
struct OpMax {
    __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
    __device__ __forceinline__ int operator()(int a, int b) const { return a > b ? a : b; }
    __device__ __forceinline__ unsigned long long operator()(unsigned long long a, unsigned long long b) const {
        return a > b ? a : b;
    }
};

template <typename V, typename Op>
__device__ __forceinline__ V warp_reduce(V v, Op op) {
#pragma unroll
    for (int width = 32; width > 1; width >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, width >> 1));
    return v;
}

// Over the block (blockDim.x a multiple of 32, at most 1024).  `sh` holds 32 values of V;
// `neutral` fills the places of warps the block does not have.
template <typename V, typename Op>
__device__ __forceinline__ V block_reduce(V v, V* sh, Op op, V neutral) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    v = warp_reduce(v, op);
    __syncthreads();              // `sh` may still be read by a reduction before this one
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    return warp_reduce(lane < n_warps ? sh[lane] : neutral, op);
}

__device__ __forceinline__ float warp_sum(float v) { return warp_reduce(v, OpSum()); }
__device__ __forceinline__ float warp_max(float v) { return warp_reduce(v, OpMax()); }
__device__ __forceinline__ float block_sum(float v, float* sh) { return block_reduce(v, sh, OpSum(), 0.f); }
__device__ __forceinline__ float block_max(float v, float* sh) { return block_reduce(v, sh, OpMax(), -INFINITY); }

// The paged cache of one run-order entry.  A page holds `page_size` positions of every kv
// head, K then V: [2][kv_heads][page_size][head_dim].  A sequence's logical page
// (pos / page_size) % ring_pages is found in its row of the page table.
struct PagedCache {
    void* base;                 // first page of this entry
    const int32_t* page_table;  // [slots][table_stride]
    int64_t page_stride;        // elements between consecutive pages
    int32_t table_stride;
    int32_t ring_pages;         // logical pages wrap at this count (= table_stride for a full cache)
    int32_t page_size;
    int32_t kv_heads;
    int32_t head_dim;
    int32_t n_pages;            // pages in the pool, for the bounds check
};

// Element offset of (slot, pos, kv head, which = 0 for K / 1 for V); -1 if there is no page, or if
// the slot is negative (a padding row that belongs to no sequence).
__device__ __forceinline__ int64_t cache_row_offset(const PagedCache& c, int slot, int pos, int kv_head, int which) {
    if (slot < 0 || pos < 0) return -1;
    const int lp = (pos / c.page_size) % c.ring_pages;
    const int page = c.page_table[(int64_t)slot * c.table_stride + lp];
    if (page < 0 || page >= c.n_pages) return -1;
    return (int64_t)page * c.page_stride +
           (((int64_t)which * c.kv_heads + kv_head) * c.page_size + (pos % c.page_size)) * c.head_dim;
}
