"""Each part of a layer alone against its plain function, and a toy mixer with state of its own that is
registered, built and stepped without a change to the library's files."""
import numpy as np
import pytest
import torch

import plain_impl as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_ctx(engine_dtype, n_rows, slots, positions, cache, decode=False):
    from x0ne_engine_b200.engine import StepContext, Workspace
    from x0ne_engine_b200.csrc import ops
    ws = Workspace(max(64, n_rows), DEV)
    ws.max_want = ws.max_rows
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)   # noqa: E731
    tr = ops.attention_prefill_tile_rows()
    return StepContext(n_rows=n_rows, tokens=mk([0] * n_rows), row_slot=mk(slots), row_pos=mk(positions),
                       dtype=engine_dtype, ws=ws, cache=cache, decode=decode, n_seqs=1, max_seq_rows=n_rows,
                       max_context=max(positions) + 1, seq_first_row=mk([0, n_rows]), seq_slot=mk(slots[:1]),
                       seq_pos0=mk(positions[:1]), n_tiles=(n_rows + tr - 1) // tr,
                       tile_seq=mk([0] * ((n_rows + tr - 1) // tr)), tile_row0=mk(list(range(0, n_rows, tr))),
                       sm_count=torch.cuda.get_device_properties(0).multi_processor_count)


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from x0ne_engine_b200.config import PartSpec
    from x0ne_engine_b200.parts import NORMS, BuildEnv
    spec = PartSpec("rmsnorm", dict(size=120, eps=3e-6, names=dict(weight="w")))
    part = NORMS.get("rmsnorm")(spec, BuildEnv(dtype, torch.device(DEV)))
    assert [(n.name, n.shape, n.role) for n in part.tensor_needs(spec)] == [("w", (120,), "vector")]
    w = 1 + 0.1 * rnd((120,), 1)
    part.bind({"w": w.to(DEV)})
    resid, delta = rnd((4, 120), 2).to(DEV), rnd((4, 120), 3).to(dtype).to(DEV)
    out = torch.empty((4, 120), dtype=dtype, device=DEV)
    want = P.rmsnorm((resid.double() + delta.double()).cpu().numpy(), w.double().numpy(), 3e-6)
    part.add_norm(None, resid, delta, out, 4)
    tol = 2e-5 if dtype == torch.float32 else 2 ** -7
    assert np.abs(out.double().cpu().numpy() - want).max() / np.abs(want).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from x0ne_engine_b200.config import PartSpec
    from x0ne_engine_b200.parts import FEED_FORWARDS, BuildEnv
    h, inter, n = 96, 200, 5
    spec = PartSpec("swiglu", dict(hidden_size=h, intermediate_size=inter, names=dict(gate="g", up="u", down="d")))
    part = FEED_FORWARDS.get("swiglu")(spec, BuildEnv(dtype, torch.device(DEV)))
    w = {"g": rnd((inter, h), 1, 0.1).to(dtype), "u": rnd((inter, h), 2, 0.1).to(dtype), "d": rnd((h, inter), 3, 0.1).to(dtype)}
    part.bind({k: v.to(DEV) for k, v in w.items()})
    x = rnd((n, h), 4).to(dtype)
    ctx = make_ctx(dtype, n, [0] * n, list(range(n)), None)
    xb = ctx.ws.buffer("x", (ctx.ws.max_rows, h), dtype)
    xb[:n] = x.to(DEV)
    out = part.forward(ctx, xb, n)[:n]
    want = P.swiglu_mlp(x.double().numpy(), {"p.gate_proj.weight": w["g"].double().numpy(),
                                             "p.up_proj.weight": w["u"].double().numpy(),
                                             "p.down_proj.weight": w["d"].double().numpy()}, "p.")
    tol = 2e-5 if dtype == torch.float32 else 3 * 2 ** -7
    assert np.abs(out.double().cpu().numpy() - want).max() / np.abs(want).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 5])
def test_attention_part_whole_then_token_by_token(dtype, window):
    """The mixer alone over its own cache group: a 70-token sequence whole, then continued one
    token at a time, against the plain attention block; with and without a window."""
    from x0ne_engine_b200.cache import SequenceCache
    from x0ne_engine_b200.config import PartSpec
    from x0ne_engine_b200.parts import MIXERS, POSITIONS, BuildEnv
    h, qh, kvh, hd, n = 72, 6, 2, 16, 75
    env = BuildEnv(dtype, torch.device(DEV))
    env.positions["p"] = POSITIONS.get("rope")(PartSpec("rope", dict(head_dim=hd, rotary_dim=hd, theta=1e4)), env)
    names = dict(q="a.q_proj.weight", k="a.k_proj.weight", v="a.v_proj.weight", o="a.o_proj.weight",
                 q_norm="a.q_norm.weight", k_norm="a.k_norm.weight")
    spec = PartSpec("gqa_attention", dict(hidden_size=h, q_heads=qh, kv_heads=kvh, head_dim=hd, qk_norm_eps=1e-5,
                                          window=window, position="p", scale=None, names=names))
    cls = MIXERS.get("gqa_attention")
    part = cls(spec, env)
    w = {"a.q_proj.weight": rnd((qh * hd, h), 1, 0.2), "a.k_proj.weight": rnd((kvh * hd, h), 2, 0.2),
         "a.v_proj.weight": rnd((kvh * hd, h), 3, 0.2), "a.o_proj.weight": rnd((h, qh * hd), 4, 0.2),
         "a.q_norm.weight": 1 + 0.1 * rnd((hd,), 5), "a.k_norm.weight": 1 + 0.1 * rnd((hd,), 6)}
    w = {k: (v.to(dtype).float() if v.dim() == 2 else v) for k, v in w.items()}
    part.bind({k: (v.to(dtype) if v.dim() == 2 else v).to(DEV) for k, v in w.items()})
    need = cls.cache_need(spec)
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("kv", kvh, hd, window)
    cache = SequenceCache([need], [None], 256, 256, dtype, DEV)
    slot = cache.acquire(n)
    x = rnd((n, h), 7).to(dtype)
    cfg = dict(q_heads=qh, kv_heads=kvh, head_dim=hd, eps=1e-5, theta=1e4)
    want = P.attention_block(x.double().numpy(), {k: v.double().numpy() for k, v in w.items()}, "a.", cfg,
                             np.arange(n), window=window)
    head = 70
    ctx = make_ctx(dtype, head, [slot] * head, list(range(head)), cache)
    xb = ctx.ws.buffer("x", (ctx.ws.max_rows, h), dtype)
    xb[:head] = x[:head].to(DEV)
    got = [part.forward(ctx, 0, xb, head)[:head].double().cpu().numpy()]
    for p in range(head, n):
        ctx = make_ctx(dtype, 1, [slot], [p], cache, decode=True)
        xb = ctx.ws.buffer("x", (ctx.ws.max_rows, h), dtype)
        xb[:1] = x[p:p + 1].to(DEV)
        got.append(part.forward(ctx, 0, xb, 1)[:1].double().cpu().numpy())
    got = np.concatenate(got)
    tol = 2e-5 if dtype == torch.float32 else 4 * 2 ** -7
    assert np.abs(got - want).max() / np.abs(want).max() < tol


def test_a_toy_mixer_with_state_of_its_own_is_registered_built_and_stepped():
    """A mixer defined here keeps a running, decayed sum of its inputs per sequence (a fixed-size
    state, no keys or values).  With a toy architecture around it the engine must build it, give it a
    zeroed state per slot, and produce the same logits whole, token by token, and after slot reuse."""
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.parts import MIXERS, CacheNeed, Mixer
    from x0ne_engine_b200.weights import RandomInit, TensorNeed, make_tensor

    class DecayMixer(Mixer):
        """state_t = decay * state_{t-1} + x_t ;  out_t = state_t @ W^T"""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.h, self.decay = int(spec["hidden_size"]), float(spec["decay"])

        @staticmethod
        def cache_need(spec):
            return CacheNeed("state", state_shape=(int(spec["hidden_size"]),))

        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec["names"]["w"], (int(spec["hidden_size"]),) * 2)]

        def bind(self, tensors):
            self.w = tensors[self.spec["names"]["w"]]

        def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
            state = ctx.cache.state(entry)
            out = ctx.ws.buffer("delta", (ctx.ws.max_rows, self.h), self.env.dtype)
            slots = ctx.row_slot[:n_rows].tolist()
            for r in range(n_rows):                      # a toy: rows in order, one at a time
                s = slots[r]
                state[s] = self.decay * state[s] + x[r].float()
                out[r] = (state[s] @ self.w.float().T).to(self.env.dtype)
            return out

    MIXERS.register("toy_decay", DecayMixer)
    try:
        h, vocab = 32, 50
        norm = lambda name: PartSpec("rmsnorm", dict(size=h, eps=1e-6, names=dict(weight=name)))   # noqa: E731
        layers = []
        for l in range(2):
            layers.append(LayerSpec(block="prenorm", parts=dict(
                mixer_norm=norm(f"l{l}.n1"),
                mixer=PartSpec("toy_decay", dict(hidden_size=h, decay=0.5 + 0.2 * l, names=dict(w=f"l{l}.mix"))),
                ffn_norm=norm(f"l{l}.n2"),
                ffn=PartSpec("swiglu", dict(hidden_size=h, intermediate_size=48,
                                            names=dict(gate=f"l{l}.g", up=f"l{l}.u", down=f"l{l}.d"))))))
        spec = ModelSpec(architecture="ToyForCausalLM", vocab_size=vocab, hidden_size=h, max_position_embeddings=64,
                         embedding=PartSpec("token_embedding", dict(vocab_size=vocab, hidden_size=h, names=dict(weight="emb"))),
                         positions={}, layers=tuple(layers), run_order=(RunEntry(0), RunEntry(1), RunEntry(0)),
                         final_norm=norm("fn"),
                         head=PartSpec("lm_head", dict(vocab_size=vocab, hidden_size=h, tied=True, names=dict(weight="emb"))))
        needs = tensor_needs_of_spec(spec)
        assert "l1.mix" in [n.name for n in needs]
        init = RandomInit(seed=3, linear_std=0.3, norm_jitter=0.1)
        cpu = {n.name: make_tensor(n, init, torch.float32, "cpu") for n in needs}
        eng = Engine(spec, {k: v.to(DEV) for k, v in cpu.items()}, "float32", DEV, max_tokens=256)
        # layer 0 runs twice (entries 0 and 2), each entry with a state of its own
        assert sorted(eng.cache.states) == [0, 1, 2] and eng.cache.state(0).data_ptr() != eng.cache.state(2).data_ptr()

        def plain(ids):
            w = {k: v.double().numpy() for k, v in cpu.items()}
            x = w["emb"][ids]
            for (l, decay) in ((0, 0.5), (1, 0.7), (0, 0.5)):
                nx = P.rmsnorm(x, w[f"l{l}.n1"], 1e-6)
                st, outs = np.zeros(h), []
                for t in range(len(ids)):
                    st = decay * st + nx[t]
                    outs.append(st @ w[f"l{l}.mix"].T)
                x = x + np.stack(outs)
                nx = P.rmsnorm(x, w[f"l{l}.n2"], 1e-6)
                x = x + P.swiglu_mlp(nx, {"p.gate_proj.weight": w[f"l{l}.g"], "p.up_proj.weight": w[f"l{l}.u"],
                                          "p.down_proj.weight": w[f"l{l}.d"]}, "p.")
            return P.rmsnorm(x, w["fn"], 1e-6) @ w["emb"].T

        ids = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9]
        want = plain(ids)
        for round_ in range(2):                           # the second round reuses the slot: state must start at zero
            s = eng.new_sequence()
            got = eng.step([s], [ids], [list(range(len(ids)))]).cpu().numpy()
            eng.free_sequence(s)
            assert np.abs(got - want).max() / np.abs(want).max() < 1e-4
        s = eng.new_sequence()
        rows = [eng.step([s], [ids[:4]], [[3]]).cpu().numpy()[0]]
        rows += [eng.step([s], [[t]]).cpu().numpy()[0] for t in ids[4:]]
        eng.free_sequence(s)
        assert np.abs(np.stack(rows) - want[3:]).max() / np.abs(want).max() < 1e-4
        # The toy reads its rows' slots back on the host, so it does not promise to be replayable:
        # the engine then pads no pass and captures no graph, and the generation loop (asked for
        # graphs, as by default) launches every step itself.  Greedy tokens in bfloat16 follow the
        # plain recurrence where its two best logits are clearly apart.
        from x0ne_engine_b200 import Model
        assert not DecayMixer.replayable and not eng.replayable
        from x0ne_engine_b200.weights.loader import held_dtype
        held = {n.name: cpu[n.name].to(DEV).to(held_dtype(n, torch.float32, torch.bfloat16)) for n in needs}
        eng16 = Engine(spec, held, "bfloat16", DEV, max_tokens=256)
        model = Model(eng16, max_batch=2)
        prompts = [ids[:7], [ids[i] for i in (4, 1, 0, 8, 2, 6, 3, 5, 7, 9, 1, 2)]]    # 7 and 12 rows
        out = model.generate(prompts, max_tokens=6)
        assert eng16.pass_graph_replays == 0 and model._generator._runner.graph_replays == 0
        assert model._generator._runner.eager_steps > 0
        for prompt, toks in zip(prompts, out.tokens):
            seq = list(prompt)
            for t in toks:
                row = plain(seq)[-1]
                best = np.sort(row)[::-1]
                if best[0] - best[1] > 0.05 * np.abs(row).max():
                    assert t == int(np.argmax(row))
                seq.append(t)
    finally:
        MIXERS.unregister("toy_decay")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_can_read_another_layers_cache(dtype):
    """Run order entry 1 runs layer 1 on the keys and values entry 0 wrote (it writes none)."""
    from x0ne_engine_b200 import Engine, Qwen3Config
    from x0ne_engine_b200.config import ModelSpec, RunEntry
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    import dataclasses
    cfg = Qwen3Config(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, vocab_size=80, max_position_embeddings=128,
                      rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=True, dtype="float32")
    spec = dataclasses.replace(cfg.to_spec(), run_order=(RunEntry(0), RunEntry(1, reads_cache_of=0)))
    init = RandomInit(seed=9, linear_std=0.1, norm_jitter=0.1)
    cpu = {n.name: make_tensor(n, init, torch.float32, "cpu") for n in tensor_needs_of_spec(spec)}
    if dtype == "bfloat16":      # what a bfloat16 engine holds of float32 matrices
        cpu = {k: (v.bfloat16().float() if v.dim() == 2 else v) for k, v in cpu.items()}
    eng = Engine(spec, {k: (v.bfloat16() if dtype == "bfloat16" and v.dim() == 2 else v).to(DEV) for k, v in cpu.items()},
                 dtype, DEV, max_tokens=256)
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [0]
    w = {k: v.double().numpy() for k, v in cpu.items()}
    pc = dict(q_heads=4, kv_heads=2, head_dim=16, eps=1e-6, theta=1e4)
    ids = [5, 9, 33, 2, 71, 8, 8, 40]
    n = len(ids)
    pos = np.arange(n)
    x = w["model.embed_tokens.weight"][ids]
    # layer 0 as usual
    nx = P.rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)
    x = x + P.attention_block(nx, w, "model.layers.0.self_attn.", pc, pos)
    k0 = P.rope(P.rmsnorm((nx @ w["model.layers.0.self_attn.k_proj.weight"].T).reshape(n, 2, 16),
                          w["model.layers.0.self_attn.k_norm.weight"], 1e-6), pos, P.inv_freq(16, 1e4))
    v0 = (nx @ w["model.layers.0.self_attn.v_proj.weight"].T).reshape(n, 2, 16)
    x = x + P.swiglu_mlp(P.rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-6), w, "model.layers.0.mlp.")
    # layer 1: its own q, layer 0's keys and values
    nx = P.rmsnorm(x, w["model.layers.1.input_layernorm.weight"], 1e-6)
    q1 = P.rope(P.rmsnorm((nx @ w["model.layers.1.self_attn.q_proj.weight"].T).reshape(n, 4, 16),
                          w["model.layers.1.self_attn.q_norm.weight"], 1e-6), pos, P.inv_freq(16, 1e4))
    x = x + P.attention(q1, k0, v0).reshape(n, 64) @ w["model.layers.1.self_attn.o_proj.weight"].T
    x = x + P.swiglu_mlp(P.rmsnorm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-6), w, "model.layers.1.mlp.")
    want = P.rmsnorm(x, w["model.norm.weight"], 1e-6) @ w["model.embed_tokens.weight"].T
    s = eng.new_sequence()
    got = eng.step([s], [ids[:5]], [list(range(5))]).cpu().numpy()
    got = np.concatenate([got] + [eng.step([s], [[t]]).cpu().numpy() for t in ids[5:]])
    assert np.abs(got - want).max() / np.abs(want).max() < (1e-4 if dtype == "float32" else 0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_with_a_windowed_layer_has_two_cache_groups_and_matches_the_plain_run(dtype):
    """Layer 1 of a toy two-layer model sees only the last 40 keys.  Its keys and values live in a
    group of their own, a ring of a few pages, while layer 0 keeps everything.  A 300-token sequence
    laps that ring several times; the engine must cut the prompt into passes the ring can take and
    still give the plain implementation's logits, whole and token by token."""
    import dataclasses
    from x0ne_engine_b200 import Engine, Qwen3Config
    from x0ne_engine_b200.config import PartSpec
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.weights import RandomInit, make_tensor
    window = 40
    cfg = Qwen3Config(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, vocab_size=90, max_position_embeddings=512,
                      rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=True, dtype=dtype)
    spec = cfg.to_spec()
    l1 = spec.layers[1]
    l1 = l1.with_part("mixer", PartSpec(l1.part("mixer").kind, {**l1.part("mixer").params, "window": window}))
    spec = dataclasses.replace(spec, layers=(spec.layers[0], l1))
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    init = RandomInit(seed=11, linear_std=0.1, norm_jitter=0.1)
    cpu = {n.name: make_tensor(n, init, tdt, "cpu") for n in tensor_needs_of_spec(spec)}
    if dtype == "float32":        # see below; in bfloat16 the effect lies under the tolerance, so the data stay as they were
        cpu["model.embed_tokens.weight"][5] *= 6.0
    from x0ne_engine_b200.weights.loader import held_dtype
    dev = {n.name: cpu[n.name].to(DEV).to(held_dtype(n, tdt, tdt)) for n in tensor_needs_of_spec(spec)}
    eng = Engine(spec, dev, dtype, DEV, max_tokens=1024)
    assert len(eng.cache.groups) == 2
    full, win = sorted(eng.cache.groups, key=lambda g: g.need.window is not None)
    assert full.need.window is None and win.need.window == window and win.ring_pages < full.ring_pages
    assert eng.cache.max_chunk <= 64

    w = {k: v.double().numpy() for k, v in cpu.items()}
    pc = dict(q_heads=4, kv_heads=2, head_dim=16, eps=1e-6, theta=1e4)
    # Token 5 (its embedding row scaled up, so that it dominates the residual of its positions)
    # stands at 150, 189 and 190: position 189 still sees key 150, the window's oldest, position 190
    # must not, although that key's page is still in the ring.  The per-head norms of q and k bound
    # every score, so one key more moves the logits by about a thousandth here: ten times the 32-bit
    # tolerance.  (The kernels alone are tested on a lapped ring with a key that decides the output.)
    special = 5
    ids = np.random.default_rng(3).integers(6, 90, 300).tolist()
    for at in (150, 189, 190):
        ids[at] = special
    pos = np.arange(len(ids))

    def plain(window_of_layer_1):
        x = w["model.embed_tokens.weight"][ids]
        for l, win_l in ((0, None), (1, window_of_layer_1)):
            p = f"model.layers.{l}."
            x = x + P.attention_block(P.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-6), w, p + "self_attn.", pc, pos,
                                      window=win_l)
            x = x + P.swiglu_mlp(P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-6), w, p + "mlp.")
        return P.rmsnorm(x, w["model.norm.weight"], 1e-6) @ w["model.embed_tokens.weight"].T

    want = plain(window)
    wider = plain(window + 1)
    assert dtype != "float32" or np.abs(wider[190] - want[190]).max() > 5e-4 * np.abs(want[190]).max(), \
        "the key just outside the window does not matter enough for this test to see it"

    def close(got, ref, what):
        err = np.max(np.abs(got - ref) / np.max(np.abs(ref), axis=-1, keepdims=True))
        assert err <= (1e-4 if dtype == "float32" else 0.05), f"{what}: {err:.3e}"

    s = eng.new_sequence()
    got = eng.step([s], [ids], [list(range(len(ids)))]).cpu().numpy()
    close(got, want, "whole")
    assert len(win.pages_of[s]) == win.ring_pages and len(full.pages_of[s]) == 5
    eng.free_sequence(s)
    s = eng.new_sequence()
    rows = [eng.step([s], [ids[:230]], [[229]]).cpu().numpy()[0]]
    rows += [eng.step([s], [[t]]).cpu().numpy()[0] for t in ids[230:]]
    eng.free_sequence(s)
    close(np.stack(rows), want[229:], "token by token")
    if dtype == "float32":
        assert np.array_equal(np.stack(rows), got[229:])


def test_rope_part_alone():
    """The position encoding part owns the table of inverse frequencies and the cos/sin table; both
    equal the plain formulas in float32, also for a rotary width below the head size."""
    from x0ne_engine_b200.config import PartSpec
    from x0ne_engine_b200.parts import POSITIONS, BuildEnv
    env = BuildEnv(dtype=torch.float32, device=torch.device(DEV))
    for head_dim, rot, theta in ((48, 48, 1e4), (80, 32, 5e5)):
        part = POSITIONS.get("rope")(PartSpec("rope", dict(head_dim=head_dim, rotary_dim=rot, theta=theta)), env)
        table, width = part.rotary()
        assert width == rot and table.dtype == torch.float32 and tuple(table.shape) == (rot // 2,)
        want = P.inv_freq(rot, theta)
        assert np.abs(table.cpu().numpy() - want).max() / want.max() < 1e-6
        cs = part.cos_sin_table(300).cpu().numpy()
        assert cs.shape == (300, rot)
        ang = (np.arange(300, dtype=np.float32)[:, None] * table.cpu().numpy()[None, :]).astype(np.float64)
        assert np.abs(cs[:, :rot // 2] - np.cos(ang)).max() < 1e-6 and np.abs(cs[:, rot // 2:] - np.sin(ang)).max() < 1e-6
    with pytest.raises(ValueError):
        POSITIONS.get("rope")(PartSpec("rope", dict(head_dim=16, rotary_dim=18, theta=1e4)), env)
    assert POSITIONS.get("none")(PartSpec("none", {}), env).rotary() is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts_alone(dtype):
    """Rows of the table as float32 (an id outside the table gives zeros); logits in float32 for a
    vocabulary and a width that are no powers of two, through the small-row and the library product."""
    from x0ne_engine_b200.config import PartSpec
    from x0ne_engine_b200.parts import BuildEnv, LMHead, TokenEmbedding
    vocab, h = 203, 72
    env = BuildEnv(dtype=dtype, device=torch.device(DEV))
    table = rnd((vocab, h), 5).to(dtype).to(DEV)
    spec = PartSpec("token_embedding", dict(vocab_size=vocab, hidden_size=h, names=dict(weight="emb")))
    emb = TokenEmbedding(spec, env)
    assert [(n.name, n.shape) for n in TokenEmbedding.tensor_needs(spec)] == [("emb", (vocab, h))]
    emb.bind({"emb": table})
    toks = [0, 202, 17, 17, 500, 3]
    ctx = make_ctx(dtype, len(toks), [0] * len(toks), list(range(len(toks))), None)
    ctx.tokens = torch.tensor(toks, dtype=torch.int32, device=DEV)
    resid = torch.full((ctx.ws.max_rows, h), 7.0, device=DEV)
    emb.forward(ctx, resid, len(toks))
    want = table.float()[[0, 202, 17, 17, 0, 3]]
    want[4] = 0
    assert torch.equal(resid[:len(toks)], want) and float(resid[len(toks)].min()) == 7.0
    head = LMHead(PartSpec("lm_head", dict(vocab_size=vocab, hidden_size=h, tied=True, names=dict(weight="emb"))), env)
    head.bind({"emb": table})
    assert head.weight_bytes() == vocab * h * table.element_size()
    for n in (3, 40):                                   # 40 rows: the library product in bfloat16
        x = rnd((n, h), 6).to(dtype).to(DEV)
        logits = torch.empty((n, vocab), dtype=torch.float32, device=DEV)
        head.forward(x, logits, n)
        ref = x.double() @ table.double().T
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert float((logits.double() - ref).abs().max() / ref.abs().max()) < tol


def test_prenorm_block_alone_with_toy_parts():
    """The arrangement alone: with a mixer that doubles and a feed-forward that triples their
    inputs, and norms that are the identity, x' = x + d + 2 (x + d) and the pending delta is
    3 x': the block adds each delta in the norm that follows it and returns its own."""
    from x0ne_engine_b200.parts import BLOCKS, FeedForward, Mixer, Norm

    class Same(Norm):
        def add_norm(self, ctx, resid, delta, out, n_rows, rows=None):
            if delta is not None:
                resid[:n_rows] += delta[:n_rows].float()
            out[:n_rows] = resid[:n_rows].to(out.dtype)

    class Twice(Mixer):
        def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
            assert (entry, cache_entry, write_cache) == (5, 2, False)
            return (2 * x).clone()

    class Thrice(FeedForward):
        def forward(self, ctx, x, n_rows):
            return (3 * x).clone()

    block = BLOCKS.get("prenorm")(dict(mixer_norm=Same(None, None), mixer=Twice(None, None), ffn_norm=Same(None, None),
                                       ffn=Thrice(None, None)))
    assert len(block.parts()) == 4 and isinstance(block.parts()[1], Twice)
    n, h = 5, 24
    ctx = make_ctx(torch.float32, n, [0] * n, list(range(n)), None)
    x, d = rnd((64, h), 1).to(DEV), rnd((64, h), 2).to(DEV)
    resid = x.clone()
    out = block.forward(ctx, 5, resid, d.clone(), cache_entry=2, write_cache=False)
    mid = x[:n] + d[:n]
    assert torch.allclose(resid[:n], 3 * mid, rtol=1e-6) and torch.allclose(out[:n], 9 * mid, rtol=1e-6)
    assert torch.equal(resid[n:], x[n:])


def test_a_toy_feed_forward_with_routing_and_a_toy_position_encoding():
    """Two more kinds of part defined here and registered without touching the library: a
    feed-forward that routes every row to one of three experts by float32 router logits, and a
    position encoding that adds a learned row to the embedding (the attention then rotates nothing).
    The model built from them gives the plain result whole, token by token, and in a batch."""
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, PositionEncoding
    from x0ne_engine_b200.weights import RandomInit, TensorNeed, make_tensor

    class TopOneExperts(FeedForward):
        """e = argmax(x R^T) in float32;  out = relu(x A_e^T) B_e^T"""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.h, self.i, self.e = int(spec["hidden_size"]), int(spec["intermediate_size"]), int(spec["experts"])

        @staticmethod
        def tensor_needs(spec):
            h, i, e, nm = int(spec["hidden_size"]), int(spec["intermediate_size"]), int(spec["experts"]), spec["names"]
            return ([TensorNeed(nm["router"], (e, h))] + [TensorNeed(f"{nm['experts']}.{k}.a", (i, h)) for k in range(e)]
                    + [TensorNeed(f"{nm['experts']}.{k}.b", (h, i)) for k in range(e)])

        def bind(self, tensors):
            nm = self.spec["names"]
            self.router = tensors[nm["router"]]
            self.a = torch.stack([tensors[f"{nm['experts']}.{k}.a"] for k in range(self.e)])
            self.b = torch.stack([tensors[f"{nm['experts']}.{k}.b"] for k in range(self.e)])

        def forward(self, ctx, x, n_rows):
            out = ctx.ws.buffer("delta", (ctx.ws.max_rows, self.h), self.env.dtype)
            xs = x[:n_rows].float()
            pick = (xs @ self.router.float().T).argmax(-1)
            hid = torch.relu(torch.einsum("rh,rih->ri", xs, self.a[pick].float()))
            out[:n_rows] = torch.einsum("ri,rhi->rh", hid, self.b[pick].float()).to(self.env.dtype)
            return out

    class LearnedPositions(PositionEncoding):
        @staticmethod
        def tensor_needs(spec):
            return [TensorNeed(spec["names"]["table"], (int(spec["positions"]), int(spec["hidden_size"])))]

        def bind(self, tensors):
            self.rows = tensors[self.spec["names"]["table"]]

        def on_embedding(self, ctx, resid, n_rows):
            resid[:n_rows] += self.rows[ctx.row_pos[:n_rows].long()].float()

    FEED_FORWARDS.register("toy_top_one", TopOneExperts)
    POSITIONS.register("toy_learned", LearnedPositions)
    try:
        h, vocab, heads, kvh, hd, inter, experts = 40, 61, 4, 2, 16, 24, 3
        norm = lambda name: PartSpec("rmsnorm", dict(size=h, eps=1e-5, names=dict(weight=name)))   # noqa: E731
        layers = []
        for l in range(2):
            att = PartSpec("gqa_attention", dict(hidden_size=h, q_heads=heads, kv_heads=kvh, head_dim=hd, qk_norm_eps=None,
                                                 window=None, position=None, scale=None,
                                                 names=dict(q=f"l{l}.q", k=f"l{l}.k", v=f"l{l}.v", o=f"l{l}.o")))
            ffn = PartSpec("toy_top_one", dict(hidden_size=h, intermediate_size=inter, experts=experts,
                                               names=dict(router=f"l{l}.router", experts=f"l{l}.experts")))
            layers.append(LayerSpec(block="prenorm", parts=dict(mixer_norm=norm(f"l{l}.n1"), mixer=att,
                                                                ffn_norm=norm(f"l{l}.n2"), ffn=ffn)))
        spec = ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=vocab, hidden_size=h, max_position_embeddings=64,
                         embedding=PartSpec("token_embedding", dict(vocab_size=vocab, hidden_size=h, names=dict(weight="emb"))),
                         positions={"learned": PartSpec("toy_learned", dict(positions=64, hidden_size=h, names=dict(table="pos")))},
                         layers=tuple(layers), run_order=(RunEntry(0), RunEntry(1)), final_norm=norm("fn"),
                         head=PartSpec("lm_head", dict(vocab_size=vocab, hidden_size=h, tied=False, names=dict(weight="head"))))
        needs = tensor_needs_of_spec(spec)
        assert {"pos", "l0.router", "l1.experts.2.b"} <= {n.name for n in needs}
        init = RandomInit(seed=11, linear_std=0.25, norm_jitter=0.1)
        cpu = {n.name: make_tensor(n, init, torch.float32, "cpu") for n in needs}
        eng = Engine(spec, {k: v.to(DEV) for k, v in cpu.items()}, "float32", DEV, max_tokens=512)
        w = {k: v.double().numpy() for k, v in cpu.items()}

        def plain(ids):
            n = len(ids)
            x = w["emb"][ids] + w["pos"][:n]
            used = set()
            for l in range(2):
                nx = P.rmsnorm(x, w[f"l{l}.n1"], 1e-5)
                q = (nx @ w[f"l{l}.q"].T).reshape(n, heads, hd)
                k = (nx @ w[f"l{l}.k"].T).reshape(n, kvh, hd)
                v = (nx @ w[f"l{l}.v"].T).reshape(n, kvh, hd)
                x = x + P.attention(q, k, v).reshape(n, heads * hd) @ w[f"l{l}.o"].T
                nx = P.rmsnorm(x, w[f"l{l}.n2"], 1e-5)
                pick = (nx @ w[f"l{l}.router"].T).argmax(-1)
                used |= set(pick.tolist())
                x = x + np.stack([np.maximum(nx[t] @ w[f"l{l}.experts.{e}.a"].T, 0) @ w[f"l{l}.experts.{e}.b"].T
                                  for t, e in enumerate(pick)])
            return P.rmsnorm(x, w["fn"], 1e-5) @ w["head"].T, used

        a, b = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 60], [1, 1, 2, 3, 5, 8, 13]
        want_a, used = plain(a)
        want_b, _ = plain(b)
        assert len(used) > 1                              # the router really sends rows to different experts
        sa, sb = eng.new_sequence(), eng.new_sequence()
        got = eng.step([sa, sb], [a[:6], b[:3]], [list(range(6)), list(range(3))]).cpu().numpy()
        assert np.abs(got[:6] - want_a[:6]).max() / np.abs(want_a).max() < 1e-4
        assert np.abs(got[6:] - want_b[:3]).max() / np.abs(want_b).max() < 1e-4
        for t in range(3, len(b)):                        # one token each; the shorter request ends first
            got = eng.step([sa, sb], [[a[3 + t]], [b[t]]]).cpu().numpy()
            assert np.abs(got[0] - want_a[3 + t]).max() / np.abs(want_a).max() < 1e-4
            assert np.abs(got[1] - want_b[t]).max() / np.abs(want_b).max() < 1e-4
        eng.free_sequence(sb)
        for t in range(3 + len(b), len(a)):
            got = eng.step([sa], [[a[t]]]).cpu().numpy()
            assert np.abs(got[0] - want_a[t]).max() / np.abs(want_a).max() < 1e-4
        eng.free_sequence(sa)
    finally:
        FEED_FORWARDS.unregister("toy_top_one")
        POSITIONS.unregister("toy_learned")


def test_toy_arrangements_embedding_and_head_are_registered_from_here():
    """What an architecture may need beyond other mixers and feed-forwards, each defined in this
    test and registered without a change to the library: an arrangement whose mixer and
    feed-forward both read one norm's output (three roles), an arrangement without a feed-forward
    (two roles), an embedding that scales its rows, and a head that soft-caps its logits.  A model
    of one layer of each arrangement is built from a spec, checked by name like any checkpoint,
    and stepped whole, token by token and in a batch against float64."""
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.config import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.parts import BLOCKS, EMBEDDINGS, HEADS, Block, LMHead, TokenEmbedding
    from x0ne_engine_b200.weights import RandomInit, make_tensor

    class ParallelBlock(Block):
        """x += mixer(norm(x)) + ffn(norm(x)): both branches read the same normed rows."""
        ROLES = {"norm": "norm", "mixer": "mixer", "ffn": "feed_forward"}

        def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
            normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
            self.norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
            a = self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache)
            both = ctx.ws.buffer("toy.both", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
            both[:ctx.n_rows] = a[:ctx.n_rows]                 # (the mixer and the feed-forward share the "delta" buffer)
            b = self.ffn.forward(ctx, normed, ctx.n_rows)
            both[:ctx.n_rows] += b[:ctx.n_rows]
            return both

    class MixerOnlyBlock(Block):
        """x += mixer(norm(x)), nothing else."""
        ROLES = {"norm": "norm", "mixer": "mixer"}

        def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
            normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
            self.norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
            return self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache)

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, ctx, resid, n_rows):
            super().forward(ctx, resid, n_rows)
            resid[:n_rows] *= float(self.spec["scale"])

    class CappedHead(LMHead):
        def forward(self, normed, logits, n_rows):
            super().forward(normed, logits, n_rows)
            cap = float(self.spec["cap"])
            logits[:n_rows] = cap * torch.tanh(logits[:n_rows] / cap)
            return logits

    BLOCKS.register("toy_parallel", ParallelBlock)
    BLOCKS.register("toy_mixer_only", MixerOnlyBlock)
    EMBEDDINGS.register("toy_scaled_embedding", ScaledEmbedding)
    HEADS.register("toy_capped_head", CappedHead)
    try:
        h, vocab, qh, kvh, hd, inter, eps, theta, scale, cap = 48, 70, 3, 1, 16, 80, 1e-5, 1e4, 3.0, 2.0
        norm = lambda name: PartSpec("rmsnorm", dict(size=h, eps=eps, names=dict(weight=name)))   # noqa: E731
        att = lambda l: PartSpec("gqa_attention", dict(                                           # noqa: E731
            hidden_size=h, q_heads=qh, kv_heads=kvh, head_dim=hd, qk_norm_eps=eps, window=None, position="rope", scale=None,
            names={k: f"l{l}.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}))
        ffn = PartSpec("swiglu", dict(hidden_size=h, intermediate_size=inter, names=dict(gate="l0.g", up="l0.u", down="l0.d")))
        layers = (LayerSpec("toy_parallel", dict(norm=norm("l0.n"), mixer=att(0), ffn=ffn)),
                  LayerSpec("toy_mixer_only", dict(norm=norm("l1.n"), mixer=att(1))))
        spec = ModelSpec(architecture="ToyForCausalLM", vocab_size=vocab, hidden_size=h, max_position_embeddings=128,
                         embedding=PartSpec("toy_scaled_embedding", dict(vocab_size=vocab, hidden_size=h, scale=scale,
                                                                         names=dict(weight="emb"))),
                         positions={"rope": PartSpec("rope", dict(head_dim=hd, rotary_dim=hd, theta=theta))},
                         layers=layers, run_order=(RunEntry(0), RunEntry(1)), final_norm=norm("fn"),
                         head=PartSpec("toy_capped_head", dict(vocab_size=vocab, hidden_size=h, tied=False, cap=cap,
                                                               names=dict(weight="head"))))
        with pytest.raises(ConfigError, match="missing"):
            tensor_needs_of_spec(dataclasses_replace_layers(spec, (LayerSpec("toy_parallel", dict(norm=norm("l0.n"), mixer=att(0))),)))
        needs = tensor_needs_of_spec(spec)
        assert {"l0.g", "l1.q", "head", "emb"} <= {n.name for n in needs} and "l1.g" not in {n.name for n in needs}
        init = RandomInit(seed=9, linear_std=0.2, norm_jitter=0.1)
        cpu = {n.name: make_tensor(n, init, torch.float32, "cpu") for n in needs}
        eng = Engine(spec, {k: v.to(DEV) for k, v in cpu.items()}, "float32", DEV, max_tokens=512)
        assert not eng.replayable                          # the toy arrangements promise nothing about graphs

        w = {k: v.double().numpy() for k, v in cpu.items()}
        pc = dict(q_heads=qh, kv_heads=kvh, head_dim=hd, eps=eps, theta=theta)

        def attention_of(x, l, pos):
            names = {f"a.{k}_proj.weight": w[f"l{l}.{k}"] for k in "qkvo"}
            names.update({"a.q_norm.weight": w[f"l{l}.q_norm"], "a.k_norm.weight": w[f"l{l}.k_norm"]})
            return P.attention_block(x, names, "a.", pc, pos)

        def plain(ids):
            pos = np.arange(len(ids))
            x = w["emb"][ids] * scale
            n0 = P.rmsnorm(x, w["l0.n"], eps)
            x = x + attention_of(n0, 0, pos) + P.swiglu_mlp(n0, {"m.gate_proj.weight": w["l0.g"], "m.up_proj.weight": w["l0.u"],
                                                                 "m.down_proj.weight": w["l0.d"]}, "m.")
            x = x + attention_of(P.rmsnorm(x, w["l1.n"], eps), 1, pos)
            return cap * np.tanh(P.rmsnorm(x, w["fn"], eps) @ w["head"].T / cap)

        a, b = prompts_of(vocab, [40, 9], seed=4)
        wa, wb = plain(a), plain(b)
        sa, sb = eng.new_sequence(), eng.new_sequence()
        got = eng.step([sa, sb], [a[:30], b[:5]], [list(range(30)), [4]]).cpu().numpy()
        rows_a, rows_b = [got[:30]], [got[30:]]
        for t in range(4):
            got = eng.step([sa, sb], [[a[30 + t]], [b[5 + t]]]).cpu().numpy()
            rows_a.append(got[:1])
            rows_b.append(got[1:])
        eng.free_sequence(sb)
        rows_a.append(eng.step([sa], [a[34:]], [list(range(6))]).cpu().numpy())
        eng.free_sequence(sa)
        for got, want, what in ((np.concatenate(rows_a), wa, "long"), (np.concatenate(rows_b), wb[4:], "short")):
            assert np.abs(got - want).max() / np.abs(want).max() < 1e-4, what
    finally:
        BLOCKS.unregister("toy_parallel")
        BLOCKS.unregister("toy_mixer_only")
        EMBEDDINGS.unregister("toy_scaled_embedding")
        HEADS.unregister("toy_capped_head")


def dataclasses_replace_layers(spec, layers):
    import dataclasses
    return dataclasses.replace(spec, layers=tuple(layers), run_order=tuple(spec.run_order[:len(layers)]))


def prompts_of(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, n).tolist() for n in lengths]
