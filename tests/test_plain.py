"""The plain implementation against the reference project's own tiny float32 Qwen3 checkpoint and
the outputs its upstream implementation produced (tests/golden), and against itself."""
import json
import os

import numpy as np

import plain_impl as P
from helpers import golden_folder


def _golden():
    cfg, w = P.read_model(golden_folder())
    with open(os.path.join(golden_folder(), "reference.json")) as f:
        return cfg, w, json.load(f)


def test_logits_hidden_attention_match_upstream():
    cfg, w, ref = _golden()
    col = {}
    lg = P.forward(cfg, w, ref["ids"], collect=col)
    want = np.array(ref["logits"]).reshape(12, cfg["vocab"])
    # the project's own tolerances: x0ne-infer/src/decoder.rs:467-493
    assert np.max(np.abs(lg - want) / (1 + np.abs(want))) < 1e-4
    att = np.array(ref["attentions"]).reshape(cfg["layers"], cfg["q_heads"], 12, 12)
    for l in range(cfg["layers"]):
        assert np.max(np.abs(col["attentions"][l] - att[l])) < 1e-5
    hid = np.array(ref["hidden"]).reshape(cfg["layers"], 12, cfg["hidden"])
    for l in range(cfg["layers"] - 1):
        assert np.max(np.abs(col["hidden"][l] - hid[l]) / (1 + np.abs(hid[l]))) < 1e-4


def test_greedy_tokens_match_upstream():
    cfg, w, ref = _golden()
    assert P.greedy(cfg, w, ref["prompt"], len(ref["generated"])) == ref["generated"]


def test_causality_and_prefix_invariance():
    cfg, w, ref = _golden()
    full = P.forward(cfg, w, ref["ids"])
    part = P.forward(cfg, w, ref["ids"][:7])
    assert np.allclose(full[:7], part, rtol=0, atol=1e-12)


def test_rope_is_relative():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 1, 16)), rng.standard_normal((1, 1, 16))
    f = P.inv_freq(16, 10000.0)
    a = (P.rope(q, np.array([5]), f) * P.rope(k, np.array([3]), f)).sum()
    b = (P.rope(q, np.array([105]), f) * P.rope(k, np.array([103]), f)).sum()
    assert abs(a - b) < 1e-4


def test_window_attention_limits_keys():
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((9, 2, 8)) for _ in range(3))
    _, probs = P.attention(q, k, v, window=3, return_probs=True)
    for i in range(9):
        assert np.all(probs[:, i, :max(0, i - 2)] == 0) and np.all(probs[:, i, i + 1:] == 0)
        assert np.allclose(probs[:, i].sum(-1), 1)


def test_round_bf16_ties_to_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38], dtype=np.float32)
    r = P.round_bf16(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625) and r[3] == -2.5


def test_nucleus_and_draw_interval():
    row = np.log(np.array([0.5, 0.2, 0.2, 0.1]))
    keep = P.nucleus_mask(P.softmax_temperature(row, 1.0), 0.6)
    assert keep.tolist() == [True, True, False, False]
    lo, hi = P.draw_interval(row, 1.0, 0.6, 1)
    assert abs(lo - 0.5 / 0.7) < 1e-12 and abs(hi - 1.0) < 1e-12
    assert P.draw_interval(row, 1.0, 0.6, 2) == (1.0, 1.0)


def test_synthetic_ids_are_pinned():
    ids = P.synthetic_ids(6, 151936)
    assert ids == P.synthetic_ids(6, 151936) and all(0 <= i < 151936 for i in ids)
