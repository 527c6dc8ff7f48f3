// Picking the next token of every sequence on the device: greedy, temperature, nucleus.
//
// One block of 1024 threads per logits row; where the caller gives a word per row of scratch, a
// launch of many blocks per row finds each row's largest logit first (one block draws some 30 GB/s
// from memory, which made 17 us of scanning for a vocabulary of 151,936).  The pick also feeds the next decode step: it
// writes the token where that step reads it, advances the sequence's position and draw
// counter, and marks the sequence finished on a stop token or a spent budget, so token and
// position never leave the device between two steps (the library engine's decode graph ends
// with argmax into tokens[0] and a position advance: x0ne-core/runtime/src/engine.rs:495-501,
// x0ne-core/kernels/cuda/argmax.cu, advance.cu).
//
// Rules (x0ne-infer/src/sampler.rs:59-147, x0ne-core/kernels/cuda/argmax.cu:4-10):
//   * any NaN in the row: no token, the row's output is -1 and the host refuses it;
//   * temperature < 1e-7 or top_p <= 0: argmax, lowest index on ties;
//   * otherwise x_i = v_i * (1/t), e_i = expf(x_i - max x), and the token is drawn by inverse
//     CDF in index order over the kept tokens; top_p >= 1 keeps all, else the nucleus: in the
//     order (probability descending, index ascending) every token whose predecessors hold less
//     than top_p of the mass.
// The uniform for draw number c of a sequence with seed s is the top 24 bits of
// splitmix64(s + (c + 1) * 0x9E3779B97F4A7C15) / 2^24: a sequence's draws depend on its seed
// and on how many tokens it has drawn, not on its batch mates.
// Sums run in a fixed order: thread t owns the contiguous index range [t*c, (t+1)*c) and adds
// it front to back; the 1024 partial sums are combined by a fixed scan.
#include "common.cuh"

#define SB 1024

// A logit and its index as one 64-bit key whose unsigned order is "larger value first, then lower
// index": the float's bits made monotone (sign flipped for positives, all bits for negatives; -0
// counts as +0) above the index counted down from 2^31 - 1.  The argmax of a row is then a plain
// maximum, which the block takes with the common reduction.  NaNs are looked for separately.
__device__ __forceinline__ unsigned long long pick_key(float v, int i) {
    uint32_t b = __float_as_uint(v + 0.0f);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (uint32_t)(0x7fffffff - i);
}
__device__ __forceinline__ float key_value(unsigned long long key) {
    uint32_t b = (uint32_t)(key >> 32);
    b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
    return __uint_as_float(b);
}
__device__ __forceinline__ int key_index(unsigned long long key) { return 0x7fffffff - (int)(uint32_t)key; }

// Inclusive scan of one value per thread over the block; returns this thread's inclusive
// prefix, and the block total through `total`.  `sh` holds 33 floats.
__device__ __forceinline__ float block_scan(float v, float* sh, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) sh[warp] = x;
    __syncthreads();
    if (warp == 0) {
        float w = sh[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        sh[lane] = w;
        if (lane == 31) sh[32] = w;
    }
    __syncthreads();
    const float before = warp > 0 ? sh[warp - 1] : 0.f;
    *total = sh[32];
    return before + x;
}

__device__ __forceinline__ int block_scan_int(int v, int* sh, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) sh[warp] = x;
    __syncthreads();
    if (warp == 0) {
        int w = sh[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        sh[lane] = w;
        if (lane == 31) sh[32] = w;
    }
    __syncthreads();
    const int before = warp > 0 ? sh[warp - 1] : 0;
    *total = sh[32];
    return before + x;
}

__device__ __forceinline__ float uniform_of(uint64_t seed, uint32_t counter) {
    uint64_t z = seed + (uint64_t)(counter + 1u) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct SampleIO {
    const float* logits;         // [rows][ld]
    const float* temperature;    // [rows] or null (greedy)
    const float* top_p;          // [rows] or null (1)
    const uint64_t* seed;        // [rows] or null (0)
    int32_t* draw_counter;       // [rows] or null
    const int32_t* stop_ids;     // [n_stop]
    int32_t* finished;           // [rows] or null
    int32_t* budget;             // [rows] or null: tokens still allowed
    int32_t* out_token;          // [rows]: the pick, -1 for a NaN row, -2 for a row already finished
    int32_t* next_token;         // [rows] or null: where the next step reads its token
    int32_t* next_pos;           // [rows] or null: advanced by one when the token will be fed
    const int32_t* status;       // null, or one int copied to out_token[rows] (the kernels' status word)
    unsigned long long* row_best; // null, or [rows]: zero before and after; the rows' largest keys, found by row_best_kernel
    int64_t ld;
    int32_t vocab;
    int32_t n_stop;
};

#define ROW_BEST_NAN (~0ull)      // above every key: the row holds a NaN

// Block (s, row) looks at its share of the row and leaves the largest key (or ROW_BEST_NAN) in
// row_best[row] with an atomic maximum, which does not depend on the order of the blocks.
__global__ void __launch_bounds__(SB) row_best_kernel(SampleIO io) {
    __shared__ unsigned long long s_key[32];
    pdl_prologue();
    const int row = blockIdx.y, tid = threadIdx.x, part = blockIdx.x, parts = gridDim.x;
    if (io.finished && io.finished[row]) return;
    const float* x = io.logits + (int64_t)row * io.ld;
    const int V = io.vocab;
    unsigned long long best = 0ull;
    bool nan = false;
    auto look = [&](float v, int i) {
        nan |= v != v;
        const unsigned long long key = pick_key(v, i);
        best = key > best ? key : best;
    };
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = V / 4;
        const int lo = (int)(((int64_t)n4 * part) / parts), hi = (int)(((int64_t)n4 * (part + 1)) / parts);
        for (int j = lo + tid; j < hi; j += SB) {
            const float4 v = x4[j];
            look(v.x, 4 * j);
            look(v.y, 4 * j + 1);
            look(v.z, 4 * j + 2);
            look(v.w, 4 * j + 3);
        }
        if (part == 0)
            for (int i = 4 * n4 + tid; i < V; i += SB) look(x[i], i);
    } else {
        const int lo = (int)(((int64_t)V * part) / parts), hi = (int)(((int64_t)V * (part + 1)) / parts);
        for (int i = lo + tid; i < hi; i += SB) look(x[i], i);
    }
    if (nan) best = ROW_BEST_NAN;
    best = block_reduce(best, s_key, OpMax(), 0ull);
    if (tid == 0 && best != 0ull) atomicMax(io.row_best + row, best);
}

__global__ void __launch_bounds__(SB, 1) sample_kernel(SampleIO io) {
    __shared__ float shf[33];
    __shared__ int shi[33];
    __shared__ unsigned long long s_key[32];
    __shared__ int s_bi[32];
    __shared__ int s_pick;
    const int row = blockIdx.x, tid = threadIdx.x;
    // This kernel writes the next step's token and position at its very end, and kernels of the
    // next step read positions and slots before they wait for their own predecessor.  So it does
    // not let its successor start early: whatever follows starts when this kernel is complete.
    pdl_wait();
    // the word in which this library's tensor-core kernels report a wait that ran out travels to
    // the host with the picks: one more int after the last row's token
    if (row == 0 && tid == 0 && io.status) io.out_token[gridDim.x] = *io.status;
    if (io.finished && io.finished[row]) {
        if (tid == 0) io.out_token[row] = -2;
        return;      // (row_best_kernel leaves a finished row's word alone: it is still zero)
    }
    const float* x = io.logits + (int64_t)row * io.ld;
    const int V = io.vocab;

    // ---- largest logit (lowest index among equals), and whether the row holds a NaN
    // (x0ne-core/kernels/cuda/argmax.cu:4-10: a NaN anywhere means no token)
    unsigned long long best = 0ull;
    bool nan = false;
    auto look = [&](float v, int i) {
        nan |= v != v;
        const unsigned long long key = pick_key(v, i);
        best = key > best ? key : best;
    };
    // four logits per load where the row starts on a 16-byte boundary (one block scans the whole row,
    // so what it has in flight decides the time: 24 us for 151,936 logits one by one); the maximum of
    // the keys does not depend on the order they are looked at
    if (io.row_best) {      // found by the launch before this one; the word goes back to zero for the next step
        best = io.row_best[row];
        nan = best == ROW_BEST_NAN;
        __syncthreads();
        if (tid == 0) io.row_best[row] = 0ull;
    } else {
        int done = 0;
        if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            const float4* x4 = reinterpret_cast<const float4*>(x);
            const int n4 = V / 4;
            for (int j = tid; j < n4; j += SB) {
                const float4 v = x4[j];
                look(v.x, 4 * j);
                look(v.y, 4 * j + 1);
                look(v.z, 4 * j + 2);
                look(v.w, 4 * j + 3);
            }
            done = 4 * n4;
        }
        for (int i = done + tid; i < V; i += SB) look(x[i], i);
    }
    const bool any_nan = __syncthreads_or(nan);
    if (any_nan) {
        if (tid == 0) {
            io.out_token[row] = -1;
            if (io.finished) io.finished[row] = 1;
        }
        return;
    }
    best = block_reduce(best, s_key, OpMax(), 0ull);
    if (tid == 0) s_pick = key_index(best);
    __syncthreads();
    const float vmax = key_value(best);

    const float t = io.temperature ? io.temperature[row] : 0.f;
    const float top_p = io.top_p ? io.top_p[row] : 1.f;
    if (t >= 1e-7f && top_p > 0.f && V > 1) {
        const float mul = 1.0f / t;
        const float xmax = vmax * mul;
        const int c = (V + SB - 1) / SB;
        const int lo = min(V, tid * c), hi = min(V, lo + c);
        // ---- total mass
        float s = 0.f;
        for (int i = lo; i < hi; ++i) s += expf(x[i] * mul - xmax);
        float Z;
        block_scan(s, shf, &Z);
        float tau = -1.f;  // keep e > tau, plus n_tie tokens with e == tau, lowest indices first
        int n_tie = 0;
        if (top_p < 1.f) {
            // Largest tau (as float bits) with mass{e >= tau} >= top_p * Z.
            const float need = top_p * Z;
            uint32_t lo_b = 0u, hi_b = 0x3f800000u;  // e lies in [0, 1]
            while (lo_b < hi_b) {
                const uint32_t mid = lo_b + (hi_b - lo_b + 1u) / 2u;
                const float th = __uint_as_float(mid);
                float ms = 0.f;
                for (int i = lo; i < hi; ++i) {
                    const float e = expf(x[i] * mul - xmax);
                    if (e >= th) ms += e;
                }
                float mass;
                block_scan(ms, shf, &mass);
                if (mass >= need) lo_b = mid; else hi_b = mid - 1u;
            }
            tau = __uint_as_float(lo_b);
            float mg = 0.f;
            for (int i = lo; i < hi; ++i) {
                const float e = expf(x[i] * mul - xmax);
                if (e > tau) mg += e;
            }
            float mass_gt;
            block_scan(mg, shf, &mass_gt);
            n_tie = 1;
            if (tau > 0.f) {
                const float k = ceilf((need - mass_gt) / tau);
                n_tie = k < 1.f ? 1 : (k > 2.0e9f ? 2000000000 : (int)k);
            } else {
                n_tie = 0x7fffffff;
            }
        }
        // ---- kept mass per thread, tie ranks in index order
        int ties = 0;
        if (top_p < 1.f)
            for (int i = lo; i < hi; ++i) ties += expf(x[i] * mul - xmax) == tau;
        int tie_total;
        const int tie_incl = block_scan_int(ties, shi, &tie_total);
        int rank = tie_incl - ties;
        float ks = 0.f;
        for (int i = lo; i < hi; ++i) {
            const float e = expf(x[i] * mul - xmax);
            bool keep = e > tau;
            if (top_p < 1.f && e == tau) keep = rank++ < n_tie;
            if (keep) ks += e;
        }
        float Zk;
        const float incl = block_scan(ks, shf, &Zk);
        const float excl = incl - ks;
        const uint64_t seed = io.seed ? io.seed[row] : 0ull;
        const uint32_t counter = io.draw_counter ? (uint32_t)io.draw_counter[row] : 0u;
        const float target = uniform_of(seed, counter) * Zk;
        if (tid == 0) s_pick = -1;
        __syncthreads();
        if (ks > 0.f && excl <= target && target < incl) {
            float run = excl;
            int pick = -1, last_kept = -1;
            rank = tie_incl - ties;
            for (int i = lo; i < hi; ++i) {
                const float e = expf(x[i] * mul - xmax);
                bool keep = e > tau;
                if (top_p < 1.f && e == tau) keep = rank++ < n_tie;
                if (!keep) continue;
                last_kept = i;
                run += e;
                if (run > target) { pick = i; break; }
            }
            s_pick = pick >= 0 ? pick : last_kept;
        }
        __syncthreads();
        if (s_pick < 0) {
            // target fell on or past the last boundary by rounding: the last kept token.
            int last = -1;
            rank = tie_incl - ties;
            for (int i = lo; i < hi; ++i) {
                const float e = expf(x[i] * mul - xmax);
                bool keep = e > tau;
                if (top_p < 1.f && e == tau) keep = rank++ < n_tie;
                if (keep) last = i;
            }
            last = block_reduce(last, s_bi, OpMax(), -1);
            if (tid == 0) s_pick = last;
            __syncthreads();
        }
    }

    if (tid == 0) {
        const int tok = s_pick;
        io.out_token[row] = tok;
        bool stop = false;
        for (int i = 0; i < io.n_stop; ++i) stop |= io.stop_ids[i] == tok;
        if (stop) {
            if (io.finished) io.finished[row] = 1;
        } else {
            if (io.draw_counter) io.draw_counter[row] += 1;
            bool spent = false;
            if (io.budget) {
                const int b = io.budget[row] - 1;
                io.budget[row] = b;
                spent = b <= 0;
            }
            if (spent) {
                if (io.finished) io.finished[row] = 1;
            } else {
                if (io.next_token) io.next_token[row] = tok;
                if (io.next_pos) io.next_pos[row] += 1;
            }
        }
    }
}

X0NE_API int x0ne_sample(SampleIO io, int n_rows, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && io.vocab > 0 && io.ld >= io.vocab, "sample: rows %d vocab %d ld %lld", n_rows,
                 io.vocab, (long long)io.ld);
    X0NE_REQUIRE(io.logits && io.out_token, "sample: null logits or output");
    X0NE_REQUIRE(io.n_stop == 0 || io.stop_ids, "sample: %d stop ids but no list", io.n_stop);
    if (n_rows == 0) return 0;
    if (io.row_best) {
        // enough blocks per row to put about two on every SM
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int parts = sms > 0 ? (2 * sms + n_rows - 1) / n_rows : 1;
        const int most = (io.vocab + 4 * SB - 1) / (4 * SB);        // a block should have a sweep of its own
        if (parts > most) parts = most;
        if (parts < 1) parts = 1;
        X0NE_REQUIRE(n_rows <= 65535, "sample: %d rows in one launch (limit 65535)", n_rows);
        x0ne_launch(row_best_kernel, dim3(parts, n_rows), dim3(SB), 0, stream, io);
        if (cudaError_t e = cudaGetLastError()) {
            x0ne_set_error("sample: launching the search for the largest logits failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    x0ne_launch(sample_kernel, dim3(n_rows), dim3(SB), 0, stream, io);
    X0NE_LAUNCH_CHECK();
}
