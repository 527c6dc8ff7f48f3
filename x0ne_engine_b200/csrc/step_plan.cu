// Host code: the tables of one pass of a step, written straight into the pinned staging buffer.
//
// A step's rows are the tokens of all its sequences, flattened; a pass is a range [r0, r1) of
// them (the whole step, or a piece of it when the step is larger than the engine's pass).  For
// that range this fills, per row, token, cache slot and position; the wanted rows that fall into
// it; the sequences that have rows in it (their first row in the pass, slot, and the position of
// that row); and the tiles of consecutive rows of one sequence that the prefill attention works
// by.  Rows past the range up to `launch_rows` are padding: slot -1, no sequence, no tile.
// It is the per-step planning that the library engine does natively for its single sequence
// (x0ne-core/runtime/src/engine.rs:702-760: positions, row counts and the logits row of a chunk).
#include <stdint.h>

#include "common.cuh"

// stage: int32 [9][stride]: 0 tokens, 1 row slots, 2 row positions, 3 wanted rows (within the pass),
//        4 tile -> sequence, 5 tile -> first row, 6 sequence -> first row (one more entry: the end),
//        7 sequence -> slot, 8 sequence -> position of its first row in the pass.
// out:   int32 [6]: sequences in the pass, tiles, most rows one sequence brings, one more than the
//        largest position, and the range [lo, hi) of `want_sorted` that falls into the pass.
X0NE_API int x0ne_plan_pass(int n_seqs, const int32_t* slots, const int32_t* starts, const int64_t* first_row,
                            const int32_t* tokens, int64_t r0, int64_t r1, const int64_t* want_sorted, int n_want,
                            int tile_rows, int launch_rows, int32_t* stage, int64_t stride, int32_t* out) {
    X0NE_REQUIRE(n_seqs > 0 && r0 >= 0 && r1 > r0 && tile_rows > 0 && stage != nullptr && out != nullptr,
                 "plan_pass: %d sequences, rows %lld to %lld", n_seqs, (long long)r0, (long long)r1);
    const int64_t n = r1 - r0;
    X0NE_REQUIRE(launch_rows >= n && launch_rows <= stride && n_seqs + 1 <= stride, "plan_pass: %lld rows (%d launched) in a table of %lld",
                 (long long)n, launch_rows, (long long)stride);
    int32_t* tok = stage;
    int32_t* rslot = stage + stride;
    int32_t* rpos = stage + 2 * stride;
    int32_t* want = stage + 3 * stride;
    int32_t* tile_seq = stage + 4 * stride;
    int32_t* tile_row0 = stage + 5 * stride;
    int32_t* seq_first = stage + 6 * stride;
    int32_t* seq_slot = stage + 7 * stride;
    int32_t* seq_pos0 = stage + 8 * stride;

    // the first sequence with a row at or after r0 (first_row is ascending)
    int lo = 0, hi = n_seqs;
    while (lo < hi) {
        const int mid = (lo + hi) / 2;
        if (first_row[mid + 1] <= r0) lo = mid + 1; else hi = mid;
    }
    int ns = 0, n_tiles = 0, max_seq_rows = 0, max_context = 0;
    for (int i = lo; i < n_seqs && first_row[i] < r1; ++i) {
        const int64_t a = first_row[i] > r0 ? first_row[i] : r0, b = first_row[i + 1] < r1 ? first_row[i + 1] : r1;
        const int rows = (int)(b - a), local = (int)(a - r0);
        const int pos0 = starts[i] + (int)(a - first_row[i]);
        seq_first[ns] = local;
        seq_slot[ns] = slots[i];
        seq_pos0[ns] = pos0;
        for (int r = 0; r < rows; ++r) {
            tok[local + r] = tokens[a + r];
            rslot[local + r] = slots[i];
            rpos[local + r] = pos0 + r;
        }
        for (int t0 = 0; t0 < rows; t0 += tile_rows) {
            X0NE_REQUIRE(n_tiles < stride, "plan_pass: more tiles than the table holds");
            tile_seq[n_tiles] = ns;
            tile_row0[n_tiles] = local + t0;
            ++n_tiles;
        }
        if (rows > max_seq_rows) max_seq_rows = rows;
        if (pos0 + rows > max_context) max_context = pos0 + rows;
        ++ns;
    }
    seq_first[ns] = (int32_t)n;
    for (int64_t r = n; r < launch_rows; ++r) {      // padding rows
        tok[r] = 0;
        rslot[r] = -1;
        rpos[r] = 0;
    }
    // wanted rows of this pass: the range of the sorted list inside [r0, r1)
    int wlo = 0, whi = n_want;
    {
        int a = 0, b = n_want;
        while (a < b) { const int mid = (a + b) / 2; if (want_sorted[mid] < r0) a = mid + 1; else b = mid; }
        wlo = a;
        b = n_want;
        while (a < b) { const int mid = (a + b) / 2; if (want_sorted[mid] < r1) a = mid + 1; else b = mid; }
        whi = a;
    }
    X0NE_REQUIRE(whi - wlo <= stride, "plan_pass: more wanted rows than the table holds");
    for (int j = wlo; j < whi; ++j) want[j - wlo] = (int32_t)(want_sorted[j] - r0);
    out[0] = ns;
    out[1] = n_tiles;
    out[2] = max_seq_rows;
    out[3] = max_context;
    out[4] = wlo;
    out[5] = whi;
    return 0;
}
