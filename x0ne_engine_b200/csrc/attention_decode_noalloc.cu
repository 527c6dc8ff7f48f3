// Decode attention with its scratch inside the library: the entry point that allocates nothing.
// See x0ne_noalloc.h for who it is for, what it costs and the rules for callers.  It has no
// counterpart in the reference project.
//
// The kernel is the split-KV decode kernel of attention_bf16.cu, unchanged: that file is
// compiled into this library too (this module is a library of its own, so nothing is defined
// twice in one library), and the entry point below only differs in where the scratch comes from.
#include "attention_bf16.cu"
#include "fast_common.cu"
#include "x0ne_noalloc.h"

// The scratch.  In host code this name is only a stand-in for the symbol: its device address is
// looked up once per device with cudaGetSymbolAddress and that pointer is what kernels get.
static __device__ __align__(256) unsigned char g_noalloc_scratch[X0NE_NOALLOC_SCRATCH_BYTES];

#define X0NE_NOALLOC_MAX_DEVICES 64
static void* g_scratch_ptr[X0NE_NOALLOC_MAX_DEVICES];   // per device, filled by its first call

X0NE_API int64_t x0ne_noalloc_scratch_capacity() { return X0NE_NOALLOC_SCRATCH_BYTES; }

X0NE_API int x0ne_attention_decode_bf16_noalloc(const void* q, void* out, PagedCache cache, const int32_t* row_slot,
                                                const int32_t* row_pos, int n_rows, int q_heads, float scale,
                                                int window, int splits, cudaStream_t stream) {
    if (int e = check_common(cache, q_heads, "attention_decode_noalloc")) return e;
    X0NE_REQUIRE(n_rows >= 0 && n_rows <= 65535, "attention_decode_noalloc: %d rows in one launch (limit 65535)", n_rows);
    X0NE_REQUIRE(splits >= 1 && splits <= 64, "attention_decode_noalloc: %d splits (1 to 64)", splits);
    // everything the launch itself would refuse is refused here, before the counters are touched
    X0NE_REQUIRE(window >= 0, "attention_decode_noalloc: negative window");
    X0NE_REQUIRE(n_rows == 0 || (q && out && row_slot && row_pos), "attention_decode_noalloc: null q, output or row tables");
    if (n_rows == 0) return 0;
    const int64_t need =
        splits > 1 ? x0ne_attention_decode_scratch_bytes(n_rows, q_heads, cache.kv_heads, cache.head_dim, splits) : 0;
    X0NE_REQUIRE(need <= X0NE_NOALLOC_SCRATCH_BYTES,
                 "attention_decode_noalloc: %d rows x %d heads x %d splits need %lld bytes of scratch; the built-in "
                 "scratch holds %d (use fewer splits, or the entry point that takes a scratch buffer)",
                 n_rows, q_heads, splits, (long long)need, X0NE_NOALLOC_SCRATCH_BYTES);
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= X0NE_NOALLOC_MAX_DEVICES) {
        x0ne_set_error("attention_decode_noalloc: cannot tell the current device (%s, device %d)",
                       cudaGetErrorString(err), dev);
        return err != cudaSuccess ? (int)err : X0NE_ERR_ARG;
    }
    if (g_scratch_ptr[dev] == nullptr) {     // the first call on this device: look the address up
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess || p == nullptr) {
            x0ne_set_error("attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
            return err != cudaSuccess ? (int)err : X0NE_ERR_ARG;
        }
        g_scratch_ptr[dev] = p;
    }
    void* scratch = g_scratch_ptr[dev];
    if (splits > 1) {
        // The arrival counters must start at zero; the array keeps whatever an earlier (possibly
        // failed) call left, so clear them on the caller's stream.
        const int G = q_heads / cache.kv_heads, gchunks = (G + 15) / 16;
        const size_t counters = (((size_t)n_rows * cache.kv_heads * gchunks * 4 + 255) / 256) * 256;
        err = cudaMemsetAsync(scratch, 0, counters, stream);
        if (err != cudaSuccess) {
            x0ne_set_error("attention_decode_noalloc: clearing the counters failed: %s", cudaGetErrorString(err));
            return (int)err;
        }
    }
    return x0ne_attention_decode_bf16(q, out, cache, row_slot, row_pos, n_rows, q_heads, scale, window, splits,
                                      splits > 1 ? scratch : nullptr, X0NE_NOALLOC_SCRATCH_BYTES, stream);
}
