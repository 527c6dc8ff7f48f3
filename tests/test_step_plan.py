"""The native planner of a pass's tables (csrc/step_plan.cu, host code) against a NumPy restatement:
unequal sequences, passes that cut sequences mid-prompt, padding rows, wanted rows in several passes."""
import numpy as np
import pytest
import torch


def restated(slots, starts, lens, tokens, r0, r1, want_sorted, tile_rows, launch_rows, stride):
    """What a pass's tables must hold, the slow way."""
    first_row = np.concatenate([[0], np.cumsum(lens)])
    row_slot = np.repeat(slots, lens)
    row_pos = np.concatenate([np.arange(st, st + n) for st, n in zip(starts, lens)])
    n = r1 - r0
    t = np.zeros((9, stride), dtype=np.int64)
    t[0, :n], t[1, :n], t[2, :n] = tokens[r0:r1], row_slot[r0:r1], row_pos[r0:r1]
    t[1, n:launch_rows] = -1
    seqs = [i for i in range(len(slots)) if first_row[i] < r1 and first_row[i + 1] > r0]
    firsts = [max(first_row[i], r0) - r0 for i in seqs] + [n]
    tiles = [(j, firsts[j] + k) for j in range(len(seqs)) for k in range(0, firsts[j + 1] - firsts[j], tile_rows)]
    t[4, :len(tiles)] = [a for a, _ in tiles]
    t[5, :len(tiles)] = [b for _, b in tiles]
    t[6, :len(firsts)] = firsts
    t[7, :len(seqs)] = [slots[i] for i in seqs]
    t[8, :len(seqs)] = [starts[i] + max(first_row[i], r0) - first_row[i] for i in seqs]
    w = [int(r - r0) for r in want_sorted if r0 <= r < r1]
    t[3, :len(w)] = w
    lo = int(np.searchsorted(want_sorted, r0))
    cols = dict(rows=launch_rows, want=len(w), tiles=len(tiles), seqs=len(seqs))
    return t, (len(seqs), len(tiles), int(np.diff(firsts).max()), int(row_pos[r0:r1].max()) + 1, lo, lo + len(w)), cols


@pytest.mark.parametrize("seed", range(6))
def test_pass_tables_match_the_restatement(seed):
    from x0ne_engine_b200.csrc import build, ops
    try:
        build.find_nvcc()
    except build.BuildError:
        pytest.skip("nvcc is needed to build the library the planner lives in")
    rng = np.random.default_rng(seed)
    n_seqs = int(rng.integers(1, 7))
    lens = rng.integers(1, 200, n_seqs) if seed else np.ones(n_seqs, dtype=np.int64)      # seed 0: a decode step
    starts = rng.integers(0, 300, n_seqs).astype(np.int32)
    slots = rng.permutation(16)[:n_seqs].astype(np.int32)
    total = int(lens.sum())
    tokens = rng.integers(0, 1000, total).astype(np.int32)
    first_row = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    want_sorted = np.sort(rng.choice(total, size=min(total, int(rng.integers(0, 12))), replace=False)).astype(np.int64)
    tile_rows = int(rng.choice([64, 128]))
    chunk = int(rng.choice([64, 65, 100, 1 << 20]))
    stride = max(min(chunk, total), n_seqs) + 1 + 64
    for r0 in range(0, total, chunk):
        r1 = min(total, r0 + chunk)
        launch_rows = min(stride, (r1 - r0 + 15) // 16 * 16)
        stage = torch.full((9, stride), 77, dtype=torch.int32)
        got = ops.plan_pass(slots, starts, first_row, tokens, r0, r1, want_sorted, tile_rows, launch_rows, stage)
        want_t, want_out, cols = restated(slots, starts, lens, tokens, r0, r1, want_sorted, tile_rows, launch_rows, stride)
        assert got == want_out
        s = stage.numpy()
        for row, upto in ((0, r1 - r0), (1, cols["rows"]), (2, r1 - r0), (3, cols["want"]), (4, cols["tiles"]), (5, cols["tiles"]),
                          (6, cols["seqs"] + 1), (7, cols["seqs"]), (8, cols["seqs"])):
            assert np.array_equal(s[row, :upto], want_t[row, :upto]), (row, r0, r1)
    with pytest.raises(ops.KernelError, match="plan_pass"):
        ops.plan_pass(slots, starts, first_row, tokens, 0, total, want_sorted, tile_rows, total, torch.zeros((9, 1), dtype=torch.int32))
