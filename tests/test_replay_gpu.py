"""bin/trace_run as a user runs it: a subprocess fed steps on standard input.  The same requests
are replayed whole, with their last 32 tokens one by one, and in batches of unequal lengths whose
shorter requests end earlier (one batch after another on a cache that holds only one batch, so
slots and pages are used again), in float32 and bfloat16, and compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import (BF16_SELF_TOL, assert_close_bf16, assert_close_f32, model_folder, plain_logits, plain_model,
                     prompts_for)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(folder, dtype, steps, max_tokens, tmp_path, vocab, extra=()):
    from x0ne_engine_b200.engine.replay import check_manifest
    out = tmp_path / f"out_{dtype}_{len(list(tmp_path.iterdir()))}"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(max_tokens), *extra], input=text, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    man = check_manifest(str(out))                     # every file present, of its shape's length, with its SHA-256
    assert man["dtype"] == dtype and man["vocab_size"] == vocab
    assert [f["step"] for f in man["files"]] == [s["step"] for s in steps if any(e.get("want") for e in s["entries"])]
    res = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if n:
            res[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, vocab)
        else:
            assert not path.exists()
    return res


def r64(n):
    return (n + 63) // 64 * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths", [("A", [40, 100, 33, 64]), ("B", [34, 97, 200, 65, 128])])
def test_replay_three_ways(name, lengths, dtype, tmp_path):
    folder = model_folder(name, "float32" if dtype == "float32" else "bfloat16")
    cfg, _ = plain_model(folder)
    vocab = cfg["vocab"]
    reqs = {f"r{i}": ids for i, ids in enumerate(prompts_for(vocab, lengths, seed=30))}
    close = assert_close_f32 if dtype == "float32" else assert_close_bf16
    plain = {k: plain_logits(folder, v) for k, v in reqs.items()}

    # (1) each request alone and whole, one after another in ONE run: the cache holds the longest only
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
             for i, (k, v) in enumerate(reqs.items())]
    whole = run_trace(folder, dtype, steps, r64(max(lengths)), tmp_path, vocab)
    whole = {k: whole[i] for i, k in enumerate(reqs)}
    for k in reqs:
        close(whole[k], plain[k], f"{name} {k} whole")

    # (2) the last 32 tokens one by one
    steps, at = [], 0
    for k, v in reqs.items():
        head = len(v) - 32
        steps.append({"step": at, "entries": [{"id": k, "tokens": v[:head], "want": [head - 1]}], "end": []})
        at += 1
        for j, t in enumerate(v[head:]):
            steps.append({"step": at, "entries": [{"id": k, "tokens": [t], "want": [0]}],
                          "end": [k] if j == 31 else []})
            at += 1
    got = run_trace(folder, dtype, steps, r64(max(lengths)), tmp_path, vocab)
    at = 0
    for k, v in reqs.items():
        rows = np.concatenate([got[at + j] for j in range(33)])
        at += 33
        base = whole[k][len(v) - 33:]
        if dtype == "float32":
            assert np.array_equal(rows, base), f"{k}: decode differs from whole"
        else:
            assert np.max(np.abs(rows - base) / np.max(np.abs(base), axis=-1, keepdims=True)) <= BF16_SELF_TOL
        close(rows, plain[k][len(v) - 33:], f"{name} {k} last 32")

    # (3) two batches of unequal lengths, one after the other; every request's last 8 tokens are
    # decoded in the batch, so the shorter prompts' requests end while the others go on
    names = list(reqs)
    batches = [names[:2], names[2:]]
    steps, at, plan = [], 0, []
    for batch in batches:
        heads = {k: len(reqs[k]) - 8 - 3 * j for j, k in enumerate(batch)}       # unequal numbers of decode steps
        steps.append({"step": at, "entries": [{"id": k, "tokens": reqs[k][:heads[k]], "want": [heads[k] - 1]}
                                              for k in batch], "end": []})
        plan.append((at, [(k, heads[k] - 1) for k in batch]))
        at += 1
        most = max(len(reqs[k]) - heads[k] for k in batch)
        for j in range(most):
            live = [k for k in batch if heads[k] + j < len(reqs[k])]
            ends = [k for k in live if heads[k] + j == len(reqs[k]) - 1]
            steps.append({"step": at, "entries": [{"id": k, "tokens": [reqs[k][heads[k] + j]], "want": [0]}
                                                  for k in live], "end": ends})
            plan.append((at, [(k, heads[k] + j) for k in live]))
            at += 1
    room = max(sum(r64(len(reqs[k])) for k in batch) for batch in batches)
    got = run_trace(folder, dtype, steps, room, tmp_path, vocab)
    for step, rows in plan:
        for j, (k, pos) in enumerate(rows):
            if dtype == "float32":
                assert np.array_equal(got[step][j], whole[k][pos]), f"step {step} {k} position {pos}"
            close(got[step][j][None], plain[k][pos][None], f"{name} batched {k} position {pos}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_steps_cut_into_passes(dtype, tmp_path):
    """`--max-step-tokens 64`: the batch's prompts (307 rows) run as five passes that cut requests
    mid-prompt; logits are wanted in every pass.  Against the same trace run in one pass per step
    (same bits in float32) and the plain implementation; then two tokens each, decoded."""
    name, lengths = "B", [34, 97, 101, 75]
    folder = model_folder(name, "float32" if dtype == "float32" else "bfloat16")
    vocab = plain_model(folder)[0]["vocab"]
    reqs = {f"r{i}": ids for i, ids in enumerate(prompts_for(vocab, lengths, seed=31))}
    want = {k: [len(v) - 3, 0, len(v) // 2] for k, v in reqs.items()}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": v[:-2], "want": want[k]} for k, v in reqs.items()], "end": []}]
    for j in (2, 1):
        steps.append({"step": len(steps), "entries": [{"id": k, "tokens": [v[-j]], "want": [0]} for k, v in reqs.items()],
                      "end": list(reqs) if j == 1 else []})
    room = sum(r64(n) for n in lengths)
    cut = run_trace(folder, dtype, steps, room, tmp_path, vocab, extra=("--max-step-tokens", "64"))
    one = run_trace(folder, dtype, steps, room, tmp_path, vocab)
    close = assert_close_f32 if dtype == "float32" else assert_close_bf16
    for step in cut:
        if dtype == "float32":
            assert np.array_equal(cut[step], one[step]), f"step {step}: passes of 64 differ from one pass"
        else:
            assert np.max(np.abs(cut[step] - one[step]) / np.max(np.abs(one[step]), axis=-1, keepdims=True)) <= BF16_SELF_TOL
    at = 0
    for k, v in reqs.items():
        plain = plain_logits(folder, v)
        close(cut[0][at:at + 3], plain[want[k]], f"{k} prompt rows")
        at += 3
    for j, step in ((2, 1), (1, 2)):
        for i, (k, v) in enumerate(reqs.items()):
            close(cut[step][i][None], plain_logits(folder, v)[len(v) - j][None], f"{k}, {j} from the end")


def test_replay_refuses_an_unknown_architecture(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architectures": ["NopeForCausalLM"]}))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(d), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True, text=True,
                       timeout=300)
    assert r.returncode != 0 and "not served" in r.stderr
