"""The engine against the plain implementation, in float32 and bfloat16, under every cut of the work:
each request alone and whole; its last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again; long decoding;
the first tokens of a sequence; greedy and sampled generation through the entry point."""
import numpy as np
import pytest
import torch

import plain_impl as P
from helpers import (BF16_SELF_TOL, assert_close_bf16, assert_close_f32, first_difference, golden_folder, model_folder,
                     plain_logits, plain_model, prompts_for)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_engines = {}


def engine(name, dtype, max_tokens=4096, **kw):
    from x0ne_engine_b200 import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        folder = golden_folder() if name == "G" else model_folder(name, "float32" if dtype == "float32" else "bfloat16")
        _engines[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw), folder)
    return _engines[key]


def check(dtype, got, want, what):
    (assert_close_f32 if dtype == "float32" else assert_close_bf16)(got, want, what)


def same_cut(dtype, got, base, what):
    """Two cuts of the same work by the engine itself."""
    got, base = np.asarray(got), np.asarray(base)
    if dtype == "float32":
        assert np.array_equal(got, base), f"{what}: first difference at {first_difference(got, base)}"
    else:
        err = np.max(np.abs(got - base) / (np.max(np.abs(base), axis=-1, keepdims=True) + 1e-30))
        assert err <= BF16_SELF_TOL, f"{what}: {err:.3e}"


def whole(eng, ids):
    s = eng.new_sequence()
    try:
        return eng.step([s], [ids], [list(range(len(ids)))]).cpu().numpy()
    finally:
        eng.free_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [5, 11, 17, 100]), ("B", [1, 7, 30, 64, 200]), ("C", [3, 65, 129]),
                                          ("G", [12, 1, 40])])
def test_each_request_alone_and_whole(name, lengths, dtype):
    eng, folder = engine(name, dtype)
    cfg, _ = plain_model(folder)
    for ids in prompts_for(cfg["vocab"], lengths, seed=1):
        want = plain_logits(folder, ids, bf16_matrices=dtype == "bfloat16")
        check(dtype, whole(eng, ids), want, f"{name} len {len(ids)}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_reference_projects_fixture(dtype):
    import json
    import os
    eng, folder = engine("G", dtype)
    with open(os.path.join(folder, "reference.json")) as f:
        ref = json.load(f)
    want = np.array(ref["logits"]).reshape(12, 40)
    if dtype == "bfloat16":
        # the fixture's matrices are float32 with a wide init; a bfloat16 engine rounds them, so it is
        # compared with the plain run on the rounded matrices (itself checked against the fixture in float64)
        want = plain_logits(folder, ref["ids"], bf16_matrices=True)
    check(dtype, whole(eng, ref["ids"]), want, "fixture logits")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n", [("A", 100), ("B", 150), ("C", 40)])
def test_last_32_tokens_one_by_one(name, n, dtype):
    eng, folder = engine(name, dtype)
    cfg, _ = plain_model(folder)
    (ids,) = prompts_for(cfg["vocab"], [n], seed=2)
    base = whole(eng, ids)
    s = eng.new_sequence()
    head = n - 32
    rows = [eng.step([s], [ids[:head]], [[head - 1]]).cpu().numpy()[0]]
    for t in ids[head:]:
        rows.append(eng.step([s], [[t]]).cpu().numpy()[0])
    eng.free_sequence(s)
    got = np.stack(rows)
    same_cut(dtype, got, base[head - 1:], f"{name}: decode vs whole")
    check(dtype, got, plain_logits(folder, ids)[head - 1:], f"{name}: decode vs plain")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_cut_into_pieces(name, dtype):
    """Chunks of 1, 2, 63, 64, 65... tokens: every piece attends the cache the earlier ones left."""
    eng, folder = engine(name, dtype)
    cfg, _ = plain_model(folder)
    n = min(cfg["max_pos"], 230)
    (ids,) = prompts_for(cfg["vocab"], [n], seed=3)
    base = whole(eng, ids)
    s = eng.new_sequence()
    rows, at = [], 0
    for size in [1, 2, 61, 64, 1, 65, 7, 1000]:
        piece = ids[at:at + size]
        if not piece:
            break
        rows.append(eng.step([s], [piece], [list(range(len(piece)))]).cpu().numpy())
        at += len(piece)
    eng.free_sequence(s)
    same_cut(dtype, np.concatenate(rows), base, f"{name}: pieces vs whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,steps", [("A", [5, 11, 17], 8), ("B", [1, 7, 30, 64], 12), ("C", [70, 3, 129, 64, 65], 40)])
def test_unequal_batches_one_after_another_reuse_slots(name, lengths, steps, dtype):
    """Three batches in a row on a cache that only holds one of them: prompts in one step, then one
    token each; request i leaves the batch after i+2 decode steps.  Every logit row must equal the
    request's own whole-sequence run, whatever slot and pages it got."""
    need = sum((n + steps + 63) // 64 * 64 for n in lengths)
    eng, folder = engine(name, dtype, max_tokens=need)
    cfg, _ = plain_model(folder)
    for batch in range(3):
        prompts = prompts_for(cfg["vocab"], lengths, seed=10 + batch)
        conts = prompts_for(cfg["vocab"], [steps] * len(lengths), seed=20 + batch)
        leave = [min(steps, i + 2) for i in range(len(lengths))]
        slots = [eng.new_sequence() for _ in prompts]
        got = [[] for _ in prompts]
        out = eng.step(slots, prompts).cpu().numpy()
        for i in range(len(prompts)):
            got[i].append(out[i])
        live = list(range(len(prompts)))
        for k in range(steps):
            live = [i for i in live if k < leave[i]]
            if not live:
                break
            out = eng.step([slots[i] for i in live], [[conts[i][k]] for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j])
            for i in live:
                if k + 1 == leave[i]:
                    eng.free_sequence(slots[i])          # shorter requests end earlier
        assert eng.cache.slots.held() == 0
        for i, p in enumerate(prompts):
            full = p + conts[i][:leave[i]]
            base = whole(eng, full)[len(p) - 1:]
            same_cut(dtype, np.stack(got[i]), base, f"{name} batch {batch} request {i}")
            check(dtype, np.stack(got[i]), plain_logits(folder, full)[len(p) - 1:], f"{name} batch {batch} request {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [5, 70, 17, 33, 90, 60]), ("B", [1, 130, 30, 64, 7]), ("C", [70, 3, 129, 64, 65])])
@pytest.mark.parametrize("pass_rows", [64, 65, 100])
def test_a_step_larger_than_one_pass_cuts_sequences_mid_prompt(name, lengths, pass_rows, dtype):
    """With `max_step_tokens` below a step's total, the flattened rows are cut into passes at row
    numbers that fall inside prompts: a sequence's first rows run in one pass, its later rows in the
    next (from the cache the first left), wanted rows lie in several passes and are asked for out of
    order and twice.  Three batches in a row on a cache that holds one.  Every logits row must be the
    request's own alone-and-whole row (same bits in float32) and the plain implementation's; then one
    token each is decoded and compared the same way."""
    need = sum((n + 1 + 63) // 64 * 64 for n in lengths)
    eng, folder = engine(name, dtype, max_tokens=need, max_step_tokens=pass_rows)
    ref, _ = engine(name, dtype)                       # an engine that runs every step in one pass
    assert eng.max_step_tokens == pass_rows and sum(lengths) > 2 * pass_rows
    cfg, _ = plain_model(folder)
    for batch in range(3):
        prompts = prompts_for(cfg["vocab"], lengths, seed=40 + batch)
        nxt = prompts_for(cfg["vocab"], [1] * len(lengths), seed=50 + batch)
        want = []
        for i, p in enumerate(prompts):                # last place first, a middle place twice, the first place
            places = [len(p) - 1, len(p) // 2, 0, len(p) // 2] if len(p) > 2 else [len(p) - 1, 0]
            want.append(places if (i + batch) % 2 == 0 else sorted(set(places)))
        slots = [eng.new_sequence() for _ in prompts]
        got = eng.step(slots, prompts, want).cpu().numpy()
        after = eng.step(slots, nxt).cpu().numpy()
        for s in slots:
            eng.free_sequence(s)
        assert eng.cache.slots.held() == 0
        at = 0
        for i, p in enumerate(prompts):
            base = whole(ref, p + nxt[i])
            plain = plain_logits(folder, p + nxt[i], bf16_matrices=dtype == "bfloat16")
            rows = got[at:at + len(want[i])]
            at += len(want[i])
            same_cut(dtype, rows, base[want[i]], f"{name} batch {batch} request {i} prompt rows, passes of {pass_rows}")
            check(dtype, rows, plain[want[i]], f"{name} batch {batch} request {i} prompt rows vs plain")
            same_cut(dtype, after[i:i + 1], base[-1:], f"{name} batch {batch} request {i} next token")
            check(dtype, after[i:i + 1], plain[-1:], f"{name} batch {batch} request {i} next token vs plain")
        assert at == len(got)


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_with_other_stop_tokens_on_the_same_model(dtype):
    """The decode graphs of a batch size are captured once and serve every later batch: a call with
    stop tokens, then one without, then one with other stop tokens, on the same model, each against
    the free run cut at its stops (a graph that kept the first call's stop list would end rows that
    the host still holds live)."""
    from x0ne_engine_b200 import Model
    folder = model_folder("A", "float32" if dtype == "float32" else "bfloat16")
    prompts = prompts_for(plain_model(folder)[0]["vocab"], [9, 4, 21, 6], seed=28)
    fresh = Model.from_folder(folder, dtype=dtype, max_batch=4, max_ctx=128)
    free = fresh.generate(prompts, max_tokens=20, stop_token_ids=()).tokens
    m = Model.from_folder(folder, dtype=dtype, max_batch=4, max_ctx=128)
    first_stop, other_stops = free[0][2], (free[1][4], free[2][1], free[3][7])

    def cut(f, stops):
        ends = [f.index(t) for t in stops if t in f]
        return f[:min(ends)] if ends else f

    for stops in ((first_stop,), (), other_stops, tuple(range(200, 230)), (first_stop,)):
        out = m.generate(prompts, max_tokens=20, stop_token_ids=stops)
        assert out.tokens == [cut(f, stops) for f in free], f"stops {stops}"
        assert m.engine.cache.slots.held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """Hundreds of single-token steps across many pages, two sequences of different age."""
    eng, folder = engine("C", dtype)
    cfg, _ = plain_model(folder)
    a, b = prompts_for(cfg["vocab"], [600, 450], seed=4)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([sa], [a[:150]], [[]])
    rows_a, rows_b = [], []
    for k in range(450):
        out = eng.step([sa, sb], [[a[150 + k]], [b[k]]]).cpu().numpy()
        rows_a.append(out[0])
        rows_b.append(out[1])
    eng.free_sequence(sa)
    eng.free_sequence(sb)
    pa, pb = plain_logits(folder, a), plain_logits(folder, b)
    check(dtype, np.stack(rows_a[-40:]), pa[-40:], "long decode a")
    check(dtype, np.stack(rows_b[-40:]), pb[-40:], "long decode b")
    check(dtype, np.stack(rows_b[:40]), pb[:40], "first tokens of a sequence")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    eng, folder = engine("B", dtype)
    cfg, _ = plain_model(folder)
    (ids,) = prompts_for(cfg["vocab"], [6], seed=5)
    s = eng.new_sequence()
    rows = [eng.step([s], [[t]]).cpu().numpy()[0] for t in ids]
    eng.free_sequence(s)
    check(dtype, np.stack(rows), plain_logits(folder, ids), "token by token from the first")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_decides_the_logits(dtype):
    """Random weights average far keys away, so a wrong page or a dropped tile could hide.  Here one
    early token's key is made to dominate a late query (its embedding row is scaled up, and the late
    token shares it), so the late logits depend on that one far key; they must match the plain run."""
    import os
    import tempfile
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.weights import open_folder, write_file
    src_folder = model_folder("C", "float32" if dtype == "float32" else "bfloat16", linear_std=0.05)
    d = tempfile.mkdtemp(prefix="x0ne_far_")
    src = open_folder(src_folder)
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    src.close()
    special = 7
    tensors["model.embed_tokens.weight"][special] *= 6.0
    write_file(os.path.join(d, "model.safetensors"), tensors)
    with open(os.path.join(src_folder, "config.json")) as f, open(os.path.join(d, "config.json"), "w") as g:
        g.write(f.read())
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=2048)
    cfg, w = P.read_model(d)
    rng = np.random.default_rng(6)
    ids = [int(t) for t in rng.integers(8, cfg["vocab"], 700)]
    ids[130] = special                    # in page 2
    ids[-1] = special
    want = P.forward(cfg, w, ids)[-3:]
    other = list(ids)
    other[130] = 9
    assert np.abs(P.forward(cfg, w, other)[-1] - want[-1]).max() > 1e-3 * np.abs(want[-1]).max(), \
        "the far key does not matter enough for this test to see it"
    s = eng.new_sequence()
    eng.step([s], [ids[:-3]], [[]])
    got = np.stack([eng.step([s], [[t]]).cpu().numpy()[0] for t in ids[-3:]])
    eng.free_sequence(s)
    check(dtype, got, want, "far key")


def test_one_and_two_long_sequences_decode_through_several_clusters_per_kv_head():
    """With one or two sequences and thousands of keys the decode attention gives every kv head
    several thread-block clusters whose results meet in scratch.  The keys of one early page are made
    to weigh on the last query (that page holds one token whose embedding row is scaled up, and the
    last prompt token is the same one), so a lost or misplaced partial result would show.
    The plain implementation takes a minute per sequence at this length, so the 32-bit path, which
    the other tests tie to it and whose attention is the plain kernel, stands in for it on the same
    bfloat16-rounded matrices.  Through the step function at batch 2 and batch 1, and through
    generation (graph replay), whose first token must be the step function's."""
    from x0ne_engine_b200 import Engine, Model, Qwen3Config
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.parts.attention import decode_plan
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    cfg = Qwen3Config(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, vocab_size=300, max_position_embeddings=16384,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, dtype="float32")
    init = RandomInit(11, 0.05, 0.1)
    tensors = {}
    for need in tensor_needs_of_spec(cfg.to_spec()):
        t = make_tensor(need, init, torch.float32, "cuda:0")
        tensors[need.name] = t.bfloat16().float() if t.dim() == 2 else t
    special = 7
    tensors["model.embed_tokens.weight"][special] *= 6.0
    n, ctx = 8600, 8704
    rng = np.random.default_rng(12)
    a = [int(t) for t in rng.integers(8, cfg.vocab_size, n)]
    b = [int(t) for t in rng.integers(8, cfg.vocab_size, n - 777)]
    a[192:256] = [special] * 64           # page 3: the first cluster's range
    a[-1] = special
    other = list(a)
    other[192:256] = [9] * 64
    last3 = lambda ids: [len(ids) - 3, len(ids) - 2, len(ids) - 1]   # noqa: E731
    ref = Engine(cfg.to_spec(), tensors, "float32", "cuda:0", max_tokens=ctx + 64, max_seq_len=ctx)
    want = {}
    for name, ids in (("a", a), ("b", b), ("other", other)):
        s = ref.new_sequence()
        want[name] = ref.step([s], [ids], [last3(ids)]).cpu().numpy()
        ref.free_sequence(s)
    del ref
    assert np.abs(want["other"][-1] - want["a"][-1]).max() > 2e-2 * np.abs(want["a"][-1]).max(), \
        "the far page does not matter enough for this test to see it"
    held = {k: (v.bfloat16() if v.dim() == 2 else v) for k, v in tensors.items()}
    eng = Engine(cfg.to_spec(), held, "bfloat16", "cuda:0", max_tokens=2 * ctx + 128, max_seq_len=ctx)
    for batch in (1, 2):
        splits, groups = decode_plan(type("C", (), {"max_context": eng.max_seq_len, "sm_count": eng.sm_count}), batch,
                                     cfg.num_key_value_heads, cfg.num_attention_heads, cfg.head_dim)
        assert groups > 1 and splits // groups >= 2, "this engine would not take the path the test is for"
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([sa, sb], [a[:-3], b[:-3]], [[], []])
    got = [eng.step([sa, sb], [[x], [y]]).cpu().numpy() for x, y in zip(a[-3:-1], b[-3:-1])]
    eng.free_sequence(sb)
    last_a = eng.step([sa], [[a[-1]]]).cpu().numpy()[0]               # batch 1
    eng.free_sequence(sa)
    check("bfloat16", np.stack([g[0] for g in got] + [last_a]), want["a"], "long context, first sequence")
    check("bfloat16", np.stack([g[1] for g in got]), want["b"][:2], "long context, second sequence")
    m = Model(eng, max_batch=2)
    out = m.generate([a, b], max_tokens=3, stop_token_ids=())
    assert out.tokens[0][0] == int(np.argmax(last_a))
    again = m.generate([a, b], max_tokens=3, stop_token_ids=())
    assert again.tokens == out.tokens


def test_decode_graphs_follow_the_context_across_a_bucket_boundary():
    """Decode graphs are kept per (rows, context bucket), because a graph fixes how the attention
    divides its work.  An engine sized for 16,384 positions generates after a prompt of 2,040 tokens
    and a short one: the long sequence crosses 2,048 on the way, so two graphs serve the batch, and
    every token must be the step function's (up to a top-2 margin within the bfloat16 tolerance)."""
    from x0ne_engine_b200 import Engine, Model, Qwen3Config
    cfg = Qwen3Config(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, vocab_size=300, max_position_embeddings=16384,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, dtype="bfloat16")
    eng = Engine.random(cfg, seed=21, dtype="bfloat16", linear_std=0.05, norm_jitter=0.1, max_tokens=3 * 2176, max_slots=3)
    assert eng.max_seq_len == 16384
    a, b = prompts_for(cfg.vocab_size, [2040, 100], seed=31)
    m = Model(eng, max_batch=2)
    n_new = 24
    out = m.generate([a, b], max_tokens=n_new, stop_token_ids=())
    assert {k for k in m._generator._runner.graphs} >= {(2, 2048), (2, 4096)}
    for prompt, got in zip((a, b), out.tokens):
        assert len(got) == n_new
        s = eng.new_sequence()
        row = eng.step([s], [prompt]).cpu().numpy()[0]
        for t in got:
            top = np.sort(row)[-2:]
            if t != int(np.argmax(row)):
                assert top[1] - top[0] <= 2 * 0.05 * np.abs(row).max(), "a token of the replayed graphs left a clear argmax"
                break
            row = eng.step([s], [[t]]).cpu().numpy()[0]
        eng.free_sequence(s)
    assert m.generate([a, b], max_tokens=n_new, stop_token_ids=()).tokens == out.tokens


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,n_new", [("A", [5, 11, 17], 8), ("B", [1, 7, 30, 64], 12)])
@pytest.mark.parametrize("decode", ["graph", "eager"])
def test_greedy_generation_through_the_entry_point(name, lengths, n_new, decode, dtype):
    from x0ne_engine_b200 import Model
    folder = model_folder(name, "float32" if dtype == "float32" else "bfloat16")
    cfg, w = plain_model(folder)
    prompts = prompts_for(cfg["vocab"], lengths, seed=7)
    m = Model.from_folder(folder, dtype=dtype, max_batch=3, max_ctx=cfg["max_pos"], decode=decode)
    out = m.generate(prompts, max_tokens=n_new, stop_token_ids=())
    assert out.finish_reasons == ["length"] * len(prompts)
    for p, got in zip(prompts, out.tokens):
        if dtype == "float32":
            assert got == P.greedy(cfg, w, p, n_new)
        else:
            # bfloat16: equal until the plain top-2 margin is within the logit tolerance
            ids = list(p)
            for t in got:
                row = P.forward(cfg, w, ids)[-1]
                top = np.sort(row)[-2:]
                if t != int(np.argmax(row)):
                    assert top[1] - top[0] <= 2 * 0.05 * np.abs(row).max(), "a bfloat16 token left a clear argmax"
                    break
                ids.append(t)
    # a second call gives the same tokens (slots and graphs reused)
    assert m.generate(prompts, max_tokens=n_new, stop_token_ids=()).tokens == out.tokens


@pytest.mark.parametrize("dtype", DTYPES)
def test_stop_tokens_and_early_endings_in_generation(dtype):
    from x0ne_engine_b200 import Model
    folder = model_folder("A", "float32" if dtype == "float32" else "bfloat16")
    cfg, w = plain_model(folder)
    prompts = prompts_for(cfg["vocab"], [9, 4, 21, 6, 13], seed=8)
    m = Model.from_folder(folder, dtype=dtype, max_batch=4, max_ctx=128)
    free = m.generate(prompts, max_tokens=20, stop_token_ids=()).tokens
    stop = free[0][3]                                         # a token the first request emits
    out = m.generate(prompts, max_tokens=20, stop_token_ids=(stop,))
    for f, got, why in zip(free, out.tokens, out.finish_reasons):
        if stop in f:
            assert got == f[:f.index(stop)] and why == "stop"
        else:
            assert got == f and why == "length"
    assert m.engine.cache.slots.held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", ["graph", "eager"])
def test_running_one_step_ahead_changes_no_token(dtype, decode):
    """The batch runner queues the next step before the host has read the current picks.  Each
    request here stops at a token of its own (which the device does not know, so the ended rows are
    stepped once more than needed), in two batches one after the other: the tokens are those of a
    runner that waits for every step, and of the free run cut at the stop."""
    from x0ne_engine_b200 import Model, SamplingParams
    from x0ne_engine_b200.engine.decode import DeviceBatch
    from x0ne_engine_b200.engine.generate import Generator
    folder = model_folder("B", "float32" if dtype == "float32" else "bfloat16")
    prompts = prompts_for(plain_model(folder)[0]["vocab"], [9, 4, 21, 6, 13, 30], seed=18)
    m = Model.from_folder(folder, dtype=dtype, max_batch=4, max_ctx=128)
    free = m.generate(prompts, max_tokens=24, stop_token_ids=()).tokens
    params = [SamplingParams(max_tokens=24, stop_token_ids=(f[2 + 3 * i],)) for i, f in enumerate(free)]
    outs = []
    for ahead in (True, False):
        def factory():
            r = DeviceBatch(m.engine, 4, cuda_graph=decode == "graph")
            r.run_ahead = ahead
            return r
        done = Generator(m.engine, max_batch=4, runner_factory=factory).generate(prompts, params)
        outs.append([c.tokens for c in done])
        assert all(c.finish_reason == "stop" for c in done)
        assert m.engine.cache.slots.held() == 0
    assert outs[0] == outs[1]
    for f, got, q in zip(free, outs[0], params):
        assert got == f[:f.index(q.stop_token_ids[0])]


@pytest.mark.parametrize("dtype", DTYPES)
def test_sampled_generation_follows_seed_and_ignores_batch_mates(dtype):
    from x0ne_engine_b200 import Model, SamplingParams
    folder = model_folder("B", "float32" if dtype == "float32" else "bfloat16")
    cfg, w = plain_model(folder)
    prompts = prompts_for(cfg["vocab"], [1, 7, 30, 64], seed=9)
    m = Model.from_folder(folder, dtype=dtype, max_batch=4, max_ctx=256)
    params = [SamplingParams(max_tokens=12, temperature=0.7, seed=100 + i) for i in range(4)]
    a = m.generate(prompts, params=params).tokens
    assert m.generate(prompts, params=params).tokens == a
    alone = [m.generate([p], params=[q]).tokens[0] for p, q in zip(prompts, params)]
    if dtype == "float32":
        assert alone == a                                     # bit-identical logits, same draws
    b = m.generate(prompts, params=[SamplingParams(max_tokens=12, temperature=0.7, seed=200 + i) for i in range(4)]).tokens
    assert a != b
    # every drawn token lies inside the interval the plain CDF gives for the request's uniform
    for p, toks, q in zip(prompts, a, params):
        ids = list(p)
        for k, t in enumerate(toks[:4]):
            row = P.forward(cfg, w, ids)[-1]
            lo, hi = P.draw_interval(row, 0.7, 1.0, t)
            u = P.uniform_of(q.seed, k)
            slack = 1e-4 if dtype == "float32" else 0.05
            assert lo - slack <= u <= hi + slack
            ids.append(t)


def test_refused_steps_change_nothing():
    from x0ne_engine_b200 import StepError
    eng, folder = engine("A", "float32", max_tokens=128)
    s = eng.new_sequence()
    eng.step([s], [[1, 2, 3]])
    for bad in (dict(slots=[s], tokens=[[256]]), dict(slots=[s], tokens=[[]]), dict(slots=[s, s], tokens=[[1], [2]]),
                dict(slots=[s], tokens=[[1]], want=[[1]]), dict(slots=[99], tokens=[[1]]),
                dict(slots=[s], tokens=[[1] * 126])):
        with pytest.raises(StepError):
            eng.step(**bad)
    assert eng.length(s) == 3
    t = eng.new_sequence()
    with pytest.raises(StepError, match="no room"):
        eng.step([t], [[1] * 100])                            # 2 pages, 1 free
    assert eng.length(t) == 0
    eng.free_sequence(s)
    eng.free_sequence(t)


def test_library_is_loaded_and_there_is_no_cpu_path():
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.csrc import ops
    engine("A", "bfloat16")
    libs = ops.loaded_libraries()
    assert any("libx0ne_core" in p for p in libs) and any("libx0ne_fast" in p for p in libs)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine.from_folder(model_folder("A"), dtype="float32", device="cpu")


@pytest.mark.parametrize("dtype", DTYPES)
def test_layers_of_the_large_shape_against_the_plain_implementation(dtype):
    """Two layers with the sizes of the 8B shape (width 4096, 32 q heads over 8 kv heads of 128,
    feed-forward 12288; the vocabulary cut to 5,000 so that the plain run stays short), random
    weights made on the device: a prompt whole, then three tokens one by one, against the plain
    implementation on the same values.  The sizes are the ones the kernels are tuned for, which the
    tiny configurations never reach (k loops of 4096 and 12288, 32 heads, 192-row products)."""
    import plain_impl as P
    from x0ne_engine_b200 import Engine, Qwen3Config
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    cfg = Qwen3Config(hidden_size=4096, intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=5000, max_position_embeddings=4096,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, dtype="float32")
    eng = Engine.random(cfg, seed=5, dtype=dtype, device="cuda:0", linear_std=0.02, norm_jitter=0.1, max_tokens=2048)
    init = RandomInit(5, 0.02, 0.1)
    w = {}
    for need in tensor_needs_of_spec(cfg.to_spec()):       # the same values, made again and taken to the host
        t = make_tensor(need, init, torch.float32, "cuda:0")
        if dtype == "bfloat16" and t.dim() == 2:
            t = t.bfloat16().float()                       # what a bfloat16 engine holds of a float32 matrix
        w[need.name] = t.cpu().numpy()
    pc = dict(hidden=4096, inter=12288, layers=2, q_heads=32, kv_heads=8, head_dim=128, vocab=5000, eps=1e-6, theta=1e6,
              tied=False, max_pos=4096)
    ids = prompts_for(5000, [200], seed=21)[0]
    want = P.forward(pc, w, ids)
    rows = [0, 63, 64, 191, 196]
    s = eng.new_sequence()
    got = eng.step([s], [ids[:197]], [rows]).cpu().numpy()
    check(dtype, got, want[rows], "prompt of 197")
    for t in range(197, 200):
        got = eng.step([s], [[ids[t]]]).cpu().numpy()
        check(dtype, got, want[t:t + 1], f"token {t}")
    eng.free_sequence(s)
    # twelve sequences at once (three prompts, four copies each, interleaved): the products for 9 to
    # 64 rows and the decode attention in clusters run at these sizes only
    prompts = prompts_for(5000, [5, 9, 12], seed=22)
    wants = [P.forward(pc, w, p) for p in prompts]
    order = [0, 1, 2] * 4
    slots = [eng.new_sequence() for _ in order]
    eng.step(slots, [prompts[i][:-2] for i in order], [[] for _ in order])
    for back in (2, 1):
        got = eng.step(slots, [[prompts[i][-back]] for i in order]).cpu().numpy()
        for row, i in enumerate(order):
            check(dtype, got[row:row + 1], wants[i][len(prompts[i]) - back][None], f"copy {row} of prompt {i}, {back} from the end")
    for sl in slots:
        eng.free_sequence(sl)


def test_all_36_layers_of_the_large_shape_in_32_bit_against_the_plain_implementation():
    """The whole depth of the 8B shape (36 layers of width 4096, 32 q heads over 8 kv heads of 128,
    feed-forward 12288; only the vocabulary is cut, to 5,000, so that the logits stay small) on the
    true 32-bit path: a 16-token prompt with logits at its first and last place, then two tokens one
    by one, against the plain float64 implementation on the same values: within 1e-4 of each row's
    largest logit, and the same greedy token.  An error that grows with depth (a residual that is
    rounded, a norm that drifts) shows here and not in two layers.  The plain run takes its weights
    one tensor at a time from the same generator, so the host never holds the model."""
    import plain_impl as P
    from x0ne_engine_b200 import Engine, Qwen3Config
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    layers, vocab = 36, 5000
    cfg = Qwen3Config(hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=vocab, max_position_embeddings=4096,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, dtype="float32")
    init = RandomInit(7, 0.02, 0.1)
    eng = Engine.random(cfg, seed=7, dtype="float32", device="cuda:0", linear_std=0.02, norm_jitter=0.1, max_tokens=64)
    ids = prompts_for(vocab, [18], seed=24)[0]
    s = eng.new_sequence()
    got = [eng.step([s], [ids[:16]], [[0, 15]]).cpu().numpy()]
    got += [eng.step([s], [[t]]).cpu().numpy() for t in ids[16:]]
    eng.free_sequence(s)
    got = np.concatenate(got)
    del eng
    torch.cuda.empty_cache()

    needs = {n.name: n for n in tensor_needs_of_spec(cfg.to_spec())}

    class OneAtATime(dict):
        def __getitem__(self, name):
            return make_tensor(needs[name], init, torch.float32, "cuda:0").cpu().numpy()

    pc = dict(hidden=4096, inter=12288, layers=layers, q_heads=32, kv_heads=8, head_dim=128, vocab=vocab, eps=1e-6, theta=1e6,
              tied=False, max_pos=4096)
    want = P.forward(pc, OneAtATime(), ids)[[0, 15, 16, 17]]
    assert_close_f32(got, want, "36 layers in 32-bit")
    assert [int(np.argmax(r)) for r in got] == [int(np.argmax(r)) for r in want]


ODD_CONFIGS = [
    # hidden, inter, layers, q heads, kv heads, head_dim, vocab, eps, theta, tied
    (100, 172, 2, 6, 3, 80, 257, 1e-6, 1e4, True),        # width no multiple of 8: the products go to the library
    (136, 264, 1, 7, 7, 16, 1000, 2e-5, 5e5, False),      # as many kv heads as q heads
    (72, 200, 3, 10, 2, 112, 333, 1e-6, 1e6, False),      # group of five, head size 112
    (64, 96, 2, 2, 1, 144, 129, 1e-5, 1e4, True),         # head size past 128: the plain attention kernel in both dtypes
    (192, 328, 2, 12, 4, 64, 515, 1e-6, 2e4, False),      # head size 64: the tcgen05 attention kernel
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ODD_CONFIGS, ids=[f"h{c[0]}_hd{c[5]}_{c[3]}over{c[4]}" for c in ODD_CONFIGS])
def test_sizes_at_the_edges_of_what_the_kernels_take(shape, dtype):
    """Head sizes in steps of 16 up to past the tensor-core kernels' limit, odd widths and
    vocabularies, any grouping: every kernel either takes the size or hands it to one that does;
    a prompt whole, two unequal prompts in one step, then tokens one by one, against the plain run."""
    import plain_impl as P
    from x0ne_engine_b200 import Engine, Qwen3Config
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    h, inter, layers, qh, kvh, hd, vocab, eps, theta, tied = shape
    cfg = Qwen3Config(hidden_size=h, intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=qh,
                      num_key_value_heads=kvh, head_dim=hd, vocab_size=vocab, max_position_embeddings=512,
                      rms_norm_eps=eps, rope_theta=theta, tie_word_embeddings=tied, dtype="float32")
    eng = Engine.random(cfg, seed=31, dtype=dtype, device="cuda:0", linear_std=0.05, norm_jitter=0.1, max_tokens=1024)
    init = RandomInit(31, 0.05, 0.1)
    w = {}
    for need in tensor_needs_of_spec(cfg.to_spec()):
        t = make_tensor(need, init, torch.float32, "cpu")
        if dtype == "bfloat16" and t.dim() == 2:
            t = t.bfloat16().float()
        w[need.name] = t.numpy()
    pc = dict(hidden=h, inter=inter, layers=layers, q_heads=qh, kv_heads=kvh, head_dim=hd, vocab=vocab, eps=eps,
              theta=theta, tied=tied, max_pos=512)
    a, b = prompts_for(vocab, [150, 40], seed=33)
    want_a, want_b = P.forward(pc, w, a), P.forward(pc, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    got = eng.step([sa, sb], [a[:140], b[:33]], [[0, 63, 64, 127, 128, 139], [0, 32]]).cpu().numpy()
    check(dtype, got[:6], want_a[[0, 63, 64, 127, 128, 139]], "long prompt")
    check(dtype, got[6:], want_b[[0, 32]], "short prompt")
    for t in range(7):
        got = eng.step([sa, sb], [[a[140 + t]], [b[33 + t]]]).cpu().numpy()
        check(dtype, got[:1], want_a[140 + t:141 + t], f"long, token {t}")
        check(dtype, got[1:], want_b[33 + t:34 + t], f"short, token {t}")
    eng.free_sequence(sb)
    for t in range(147, 150):
        check(dtype, eng.step([sa], [[a[t]]]).cpu().numpy(), want_a[t:t + 1], f"long alone, token {t}")
    eng.free_sequence(sa)


def test_long_prompt_at_the_large_shape_bfloat16_against_the_32_bit_path():
    """1,500 tokens through two layers of the 8B shape: here the bfloat16 engine runs its
    large-pass kernels (tcgen05 attention over 12 row tiles, the fused tcgen05 gate/up product from
    768 rows), which the plain implementation is too slow to check; the 32-bit path, which the other
    tests tie to the plain implementation, stands in for it on the same bfloat16-rounded matrices."""
    from x0ne_engine_b200 import Engine, Qwen3Config
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    cfg = Qwen3Config(hidden_size=4096, intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=5000, max_position_embeddings=4096,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, dtype="float32")
    init = RandomInit(6, 0.02, 0.1)
    tensors = {}
    for need in tensor_needs_of_spec(cfg.to_spec()):
        t = make_tensor(need, init, torch.float32, "cuda:0")
        tensors[need.name] = t.bfloat16().float() if t.dim() == 2 else t
    ids = prompts_for(5000, [1503], seed=23)[0]
    rows = [0, 127, 128, 767, 768, 1023, 1499]
    got = {}
    for dtype in ("float32", "bfloat16"):
        held = {k: (v.bfloat16() if dtype == "bfloat16" and v.dim() == 2 else v) for k, v in tensors.items()}
        eng = Engine(cfg.to_spec(), held, dtype, "cuda:0", max_tokens=2048)
        s = eng.new_sequence()
        out = [eng.step([s], [ids[:1500]], [rows]).cpu().numpy()]
        out += [eng.step([s], [[t]]).cpu().numpy() for t in ids[1500:]]
        eng.free_sequence(s)
        got[dtype] = np.concatenate(out)
        del eng, held
        torch.cuda.empty_cache()
    assert_close_bf16(got["bfloat16"], got["float32"], "1,500 tokens at the large shape")


@pytest.mark.parametrize("name", ["A", "B"])
def test_short_prompt_passes_replayed_from_graphs_give_the_same_bits(name):
    """Short bfloat16 prompt passes are launched with a padded row count and, from the second pass
    of a kind on, replayed from a CUDA graph.  Against an engine that launches every pass itself:
    the same bits for the prompts' logits and for a decoded token after them (so the cache holds
    the same values), for lengths that share a graph, batches, and further pieces of a prompt."""
    eng, _ = engine(name, "bfloat16")
    base, _ = engine(name, "bfloat16", pass_graphs=False)
    assert eng.pass_graphs and not base.pass_graphs
    rounds = [[100], [120], [70], [126], [20], [30], [17], [5], [5], [6], [100, 20], [90, 30], [33, 3, 40], [35, 2, 39],
              [100], [65]]
    before = eng.pass_graph_replays
    for k, lengths in enumerate(rounds):
        prompts = prompts_for(eng.vocab_size, lengths, seed=100 + k)
        got = []
        for e in (eng, base):
            slots = [e.new_sequence() for _ in lengths]
            try:
                first = e.step(slots, prompts).cpu().numpy()
                nxt = e.step(slots, [[int(np.argmax(r))] for r in first]).cpu().numpy()
            finally:
                for s in slots:
                    e.free_sequence(s)
            got.append((first, nxt))
        assert np.array_equal(got[0][0], got[1][0]), f"prompts of {lengths}: {first_difference(got[0][0], got[1][0])}"
        assert np.array_equal(got[0][1], got[1][1]), f"token after {lengths}: {first_difference(got[0][1], got[1][1])}"
    assert eng.pass_graph_replays - before >= 6 and base.pass_graph_replays == 0
    # further pieces of a prompt: two sequences whose second pieces share a graph
    outs = []
    for e in (eng, base):
        res = []
        for a, b, seed in ((40, 30, 7), (45, 28, 8), (41, 29, 9)):
            ids = prompts_for(e.vocab_size, [a + b], seed=seed)[0]
            s = e.new_sequence()
            try:
                e.step([s], [ids[:a]], [[]])
                res.append(e.step([s], [ids[a:]]).cpu().numpy())
            finally:
                e.free_sequence(s)
        outs.append(res)
    for x, y in zip(*outs):
        assert np.array_equal(x, y)
    # and against the plain implementation, through a replayed graph
    folder = engine(name, "bfloat16")[1]
    ids = prompts_for(eng.vocab_size, [100], seed=3)[0]
    n0 = eng.pass_graph_replays
    s = eng.new_sequence()
    try:
        got = eng.step([s], [ids]).cpu().numpy()
    finally:
        eng.free_sequence(s)
    assert eng.pass_graph_replays == n0 + 1
    check("bfloat16", got, plain_logits(folder, ids, bf16_matrices=True)[-1:], "a replayed prompt pass")
