"""Command line of the library: `python -m x0ne_engine_b200 <command> ...`.

Commands and their options follow the reference's own programs where it has them:

  core-bench <model dir> [--lengths short,1k,4k,16-1024] [--decode N] [--reps N] [--batch B] [--dtype D]
      [--random-weights SEED] [--clock-trace]
      time to first token, prefill and decode rates and the gaps between tokens (p50 / p90 / p99, as
      x0ne-core/runtime/src/engine.rs:1106-1116 stamps them) per prompt length, one line
      `x0ne-bench-result: <JSON>` (x0ne-core/oracle/examples/core-bench.rs:6-16,420-436).  Exit code
      3 when two repetitions of a length gave different tokens
      (x0ne-core/oracle/examples/core-perf.rs:85-89).  A length "16-1024" is an unequal batch: prompt
      lengths uniform between the two ends, from a seed.  --clock-trace adds the SM clock during the
      last repetition (read through NVML, nothing is set): what the prompts' pass does to the clock
      and how long the first decode steps run at the lowered clock.
  roofline --config config.json --gpu <GB/s> --prompt P --generated N [--tok-s X] [--batch B]
      places a decode rate against the bandwidth ceiling
      (x0ne-core/runtime/src/bin/x0ne-core-roofline.rs:4-5, x0ne-core/runtime/src/roofline.rs:55-102).
  generate <model dir> --prompt-ids 1,2,3 [--prompt-ids ...] [--max-tokens N] [--temperature T]
      [--top-p P] [--seed S] [--stop-token-ids a,b] [--dtype D] [--decode graph|eager]
  replay ...            the trace replay program (same as bin/trace_run)
  init <config.json> <out dir> [--seed S] [--linear-std X] [--norm-jitter X]
      writes a model folder with random weights
  step-timeline <model dir> [--batch B] [--context N] [--random-weights SEED]
      one decode step of B sequences at context N as the GPU ran it: every kernel of the replayed graph
      with the time from the end of the kernel before it to its own end (what it adds to the step)
      and its own duration, summed per kernel and listed for one layer in the middle of the model
  kernel-bench --kernel NAME [sizes] [--impl ours|reference]   times one kernel alone with CUDA events
      (the reference's per-kernel timing entry: x0ne-core/runtime/src/ops.rs:579-681).  With
      `--impl reference` the reference project's own kernel of that name (attention_decode,
      attention_prefill, add_rmsnorm, qk_norm_rope, swiglu), compiled unchanged from its sources, runs
      on the same sizes at batch 1, the only batch its kernels take.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time


def _ids(text: str):
    return [int(t) for t in text.split(",") if t.strip() != ""]


def synthetic_ids(n: int, vocab: int, seed: int = 0x0C0E5EED):
    """splitmix64 ids (x0ne-core/oracle/examples/core-bench.rs:26-43)."""
    m = (1 << 64) - 1
    s, out = seed, []
    for _ in range(n):
        s = (s + 0x9E3779B97F4A7C15) & m
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        out.append(int((z ^ (z >> 31)) % vocab))
    return out


def _stats(v):
    if not v:
        return None
    s = sorted(v)
    return {"median": statistics.median(s), "min": s[0], "max": s[-1], "mean": statistics.fmean(s),
            "stddev": statistics.stdev(s) if len(s) > 1 else 0.0, "n": len(s)}


def _length_tokens(name: str, limit: int) -> int:
    if "-" in name:                      # "16-1024": an unequal batch; the longest prompt sizes the run
        return _length_tokens(name.split("-", 1)[1], limit)
    if name == "short":
        return 20
    if name == "max":
        return limit - 1
    if name.endswith("k"):
        return int(name[:-1]) * 1024
    return int(name)


def cmd_generate(a) -> int:
    from . import Model
    m = Model.from_folder(a.model, dtype=a.dtype, max_batch=max(1, len(a.prompt_ids)), max_ctx=a.max_ctx,
                          decode=a.decode)
    stop = None if a.stop_token_ids is None else tuple(_ids(a.stop_token_ids))
    out = m.generate([_ids(p) for p in a.prompt_ids], max_tokens=a.max_tokens, temperature=a.temperature,
                     top_p=a.top_p, seed=a.seed, stop_token_ids=stop)
    for toks, why in zip(out.tokens, out.finish_reasons):
        print(json.dumps({"tokens": toks, "finish_reason": why}))
    return 0


class _ClockPoll:
    """Reads the SM clock and the power draw through NVML every millisecond on a host thread
    (reading only; it sets nothing)."""

    def __init__(self, device: int = 0):
        import threading
        import pynvml
        pynvml.nvmlInit()
        self._nvml, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(device)
        self.samples, self._stop = [], False
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        n = self._nvml
        while not self._stop:
            self.samples.append((time.perf_counter(), n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM),
                                 n.nvmlDeviceGetPowerUsage(self._h) / 1000.0))
            time.sleep(0.001)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop = True
        self._thread.join()

    def runs(self, first_token_at: float, gaps) -> list:
        """Stretches of one clock value, in milliseconds after the first token (negative: during the
        prompts' pass), each with the median gap of the tokens that arrived in it."""
        arrivals, t = [], first_token_at
        for g in gaps:
            t += g
            arrivals.append((t, g))
        out = []
        for ts, mhz, watts in self.samples:
            if out and out[-1]["sm_mhz"] == mhz:
                out[-1]["_to"], out[-1]["_w"] = ts, out[-1]["_w"] + [watts]
            else:
                out.append({"sm_mhz": mhz, "_from": ts, "_to": ts, "_w": [watts]})
        for r in out:
            inside = sorted(g for t, g in arrivals if r["_from"] <= t <= r["_to"])
            r["from_ms"] = round((r.pop("_from") - first_token_at) * 1e3, 1)
            r["to_ms"] = round((r.pop("_to") - first_token_at) * 1e3, 1)
            r["watts"] = round(sorted(r["_w"])[len(r.pop("_w")) // 2])
            r["tokens"], r["gap_ms_median"] = len(inside), round(inside[len(inside) // 2] * 1e3, 3) if inside else None
        return out


def cmd_core_bench(a) -> int:
    import torch
    from . import Model
    from .config import config_from_folder
    from .engine.generate import GenerationStats, percentiles
    cfg = config_from_folder(a.model)
    limit, vocab = cfg.to_spec().max_position_embeddings, cfg.to_spec().vocab_size
    names = [n.strip() for n in a.lengths.split(",")]
    if any(not n for n in names) or a.decode < 2 or a.reps < 1:
        print("usage: core-bench <model directory> [--lengths a,b,...] [--decode N>=2] [--reps N>=1]", file=sys.stderr)
        return 2
    lens = [_length_tokens(n, limit - a.decode) for n in names]
    max_ctx = min(limit, max(lens) + a.decode)
    t0 = time.time()
    if a.random_weights is not None:      # the folder needs only its config.json
        m = Model.random(cfg, seed=a.random_weights, dtype=a.dtype, max_batch=a.batch, max_ctx=max_ctx)
    else:
        m = Model.from_folder(a.model, dtype=a.dtype, max_batch=a.batch, max_ctx=max_ctx)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    results = []
    for name, n in zip(names, lens):
        if "-" in name:                  # lengths uniform between the two ends, from the same generator as the ids
            lo = _length_tokens(name.split("-", 1)[0], limit - a.decode)
            each = [lo + v % (n - lo + 1) for v in synthetic_ids(a.batch, 1 << 30, 0x1E26)]
        else:
            each = [n] * a.batch
        prompts = [synthetic_ids(k, vocab, 0x0C0E5EED + i) for i, k in enumerate(each)]
        ttft, prefill, decode, tokens, gaps = [], [], [], [], []
        first = None
        # two runs before the timed ones: the first launches a short prompt pass itself, the second
        # captures its launches into a graph, later ones replay it
        clock_runs = None
        for rep in range(a.reps + 2):
            m._generator.stats = st = GenerationStats()
            if a.clock_trace and rep == a.reps + 1:
                time.sleep(0.5)                     # the GPU idles first, as before a user's call
                with _ClockPoll(torch.cuda.current_device()) as poll:
                    began = time.perf_counter()
                    out = m.generate(prompts, max_tokens=a.decode, stop_token_ids=())
                clock_runs = poll.runs(began + st.prefill_seconds, st.token_gaps)
            else:
                out = m.generate(prompts, max_tokens=a.decode, stop_token_ids=())
            rates = (st.prefill_seconds, st.prefill_tokens / st.prefill_seconds,
                     st.decode_tokens / st.decode_seconds if st.decode_seconds else 0.0)
            if rep == 0:
                first = rates
            elif rep >= 2:
                ttft.append(rates[0]); prefill.append(rates[1]); decode.append(rates[2]); tokens.append(out.tokens)
                gaps += st.token_gaps
        same = all(t == tokens[0] for t in tokens)
        results.append({"name": name, "tokens": n, "prompt_tokens": each, "source": "synthetic", "status": "ok" if same else "tokens differ",
                        "same_tokens": same,
                        "first": {"ttft_s": first[0], "prefill_tok_s": first[1], "decode_tok_s": first[2]},
                        "ttft_s": _stats(ttft), "prefill_tok_s": _stats(prefill), "decode_tok_s": _stats(decode),
                        "token_gap_s": percentiles(gaps)})
        if clock_runs is not None:
            results[-1]["clock_runs"] = clock_runs
    free, total = torch.cuda.mem_get_info()
    spec = m.engine.spec
    print("x0ne-bench-result: " + json.dumps({
        "schema": 1, "kind": "core", "model": a.model, "max_ctx": max_ctx, "decode_tokens": a.decode, "reps": a.reps,
        "batch": a.batch, "engine": m.engine.describe(),
        "config": {"architecture": spec.architecture, "layers": len(spec.run_order), "hidden_size": spec.hidden_size,
                   "vocab_size": spec.vocab_size, "max_position_embeddings": spec.max_position_embeddings,
                   "step_weight_bytes": m.engine.model.step_weight_bytes(),
                   "cache_bytes_per_token": m.engine.cache.bytes_per_token()},
        "load": {"cold_s": load_s}, "memory": {"device_total_bytes": total, "free_after_bytes": free},
        "lengths": results}))
    if not all(r["same_tokens"] for r in results):
        # a rate measured while the tokens change from one repetition to the next is no measurement of generation
        print("core-bench: two repetitions of the same greedy generation gave different tokens", file=sys.stderr)
        return 3
    return 0


def cmd_step_timeline(a) -> int:
    """Kernels overlap inside a step (each is launched while the one before it still runs and waits
    for it on the device), so a kernel's own duration says little; what it adds to the step is the
    time from its predecessor's end to its own end.  Taken with torch's profiler around one replay of
    the decode graph, after the step has been timed without the profiler."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    from . import Model
    from .config import config_from_folder
    from .engine.decode import DeviceBatch
    from .engine.generate import Row
    from .sampling import SamplingParams
    cfg = config_from_folder(a.model)
    spec = cfg.to_spec()
    max_ctx = min(spec.max_position_embeddings, a.context + 64)
    if a.random_weights is not None:
        m = Model.random(cfg, seed=a.random_weights, dtype="bfloat16", max_batch=a.batch, max_ctx=max_ctx)
    else:
        m = Model.from_folder(a.model, dtype="bfloat16", max_batch=a.batch, max_ctx=max_ctx)
    eng = m.engine
    plen = a.context - 8
    rows = [Row(i, synthetic_ids(plen, spec.vocab_size, 1 + i), SamplingParams(max_tokens=max_ctx), max_ctx - plen, i)
            for i in range(a.batch)]
    runner = DeviceBatch(eng, a.batch, cuda_graph=True)
    runner.run_ahead = False
    try:
        runner.start(rows)
        live = list(range(a.batch))
        for _ in range(5):
            runner.step(live)
        g = runner.last_graph
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(20):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / 20
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
        for slot in runner.slots:
            eng.cache.lengths[slot] += 23
    finally:
        runner.close()
    ev = sorted((k for k in prof.events() if k.device_type == torch.autograd.DeviceType.CUDA), key=lambda k: k.time_range.start)
    last = ev[-(len(ev) // 3):]
    weights, kv = eng.model.step_weight_bytes(), eng.cache.bytes_per_token() * a.batch * a.context
    print(f"{eng.describe()}\nbatch {a.batch}, context {a.context}: {ms:.3f} ms per step without the profiler; a step reads "
          f"{(weights + kv) / 1e9:.2f} GB = {(weights + kv) / ms / 1e6:.0f} GB/s")
    share = collections.OrderedDict()
    prev = last[0].time_range.start
    for k in last:
        name = k.name.split("(")[0][:56]
        t = share.setdefault(name, [0, 0.0, 0.0])
        t[0] += 1
        t[1] += k.time_range.end - prev
        t[2] += k.time_range.end - k.time_range.start
        prev = k.time_range.end
    print(f"one replay under the profiler: {last[-1].time_range.end - last[0].time_range.start:.0f} us, {len(last)} kernels")
    print("   adds us   launches   each   own duration each   kernel")
    for name, (n, add, own) in share.items():
        print(f"{add:10.1f} {n:10d} {add / n:6.2f} {own / n:19.2f}   {name}")
    n_entries = len(spec.run_order)
    per_layer = (len(last) - 4) // max(1, n_entries)
    start = 2 + per_layer * (n_entries // 2)
    print(f"layer {n_entries // 2} of {n_entries}:")
    prev = last[start - 1].time_range.end
    for k in last[start:start + per_layer]:
        print(f"   adds {k.time_range.end - prev:6.2f} us   own {k.time_range.end - k.time_range.start:6.2f}   {k.name[:80]}")
        prev = k.time_range.end
    return 0


def cmd_roofline(a) -> int:
    """Bytes from the model as data: every run-order entry's tensors once and the head's, and what
    one position of one sequence holds in the cache; nothing here names an architecture."""
    from .config import config_from_folder
    from .engine.model import step_bytes_of_spec
    import os
    spec = config_from_folder(os.path.dirname(os.path.abspath(a.config))).to_spec()
    weights, kv_per_position = step_bytes_of_spec(spec, 2)
    ctx = a.prompt + a.generated / 2.0
    kv = kv_per_position * ctx * a.batch
    ceiling = a.gpu * 1e9 / (weights + kv) * a.batch
    row = {"architecture": spec.architecture, "prompt_tokens": a.prompt, "generated": a.generated, "batch": a.batch,
           "mean_ctx": ctx, "weight_bytes": weights, "kv_bytes": kv, "bandwidth_gb_s": a.gpu, "ceiling_tok_s": ceiling}
    if a.tok_s is not None:
        row.update(tok_s=a.tok_s, share=a.tok_s / ceiling)
    print(json.dumps(row))
    return 0


def cmd_init(a) -> int:
    from .config import config_from_dict
    from .weights import RandomInit, write_model_folder
    with open(a.config) as f:
        cfg = config_from_dict(json.load(f))
    write_model_folder(a.out, cfg, RandomInit(a.seed, a.linear_std, a.norm_jitter))
    print(f"wrote {a.out}")
    return 0


def cmd_replay(a, rest) -> int:
    from .engine.replay import main
    return main(rest)


def cmd_kernel_bench(a) -> int:
    """Times one kernel alone: inputs larger than L2 are cycled so every launch reads cold data."""
    import math
    import torch
    from .csrc import ops
    dev = "cuda:0"
    torch.manual_seed(0)

    def timed(fn, bytes_per_launch, flops_per_launch=0.0, n_copies=None):
        """The launches are captured into one CUDA graph, so the time is the device's, not the host's."""
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(a.iters):
                fn()
        g.replay()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1e3 / a.iters
        print(json.dumps({"kernel": a.kernel, "impl": a.impl, "m": a.m, "n": a.n, "k": a.k, "batch": a.batch,
                          "context": a.context, "us": us, "gb_s": bytes_per_launch / us / 1e3, "tflops": flops_per_launch / us / 1e6,
                          "copies": copies if n_copies is None else n_copies}))

    copies = 1
    if a.impl == "reference":
        return _kernel_bench_reference(a, timed)

    if a.kernel in ("gemm_smallm", "gemm_smallm_swiglu", "gemm_library", "gemm_tc", "gemm_tc_swiglu", "gemm_tc1",
                    "gemm_tc1_swiglu", "gemm_skinny", "gemm_skinny_swiglu"):
        swiglu = a.kernel.endswith("_swiglu")
        rows = 2 * a.n if swiglu else a.n
        wbytes = rows * a.k * 2
        copies = max(2, int(math.ceil(256e6 / wbytes)) + 1)          # cycle through > 2 x L2 of weights
        ws = [torch.randn(rows, a.k, device=dev).mul_(0.02).bfloat16() for _ in range(copies)]
        x = torch.randn(max(a.m, 1), a.k, device=dev).bfloat16()
        y = torch.empty(max(a.m, 1), a.n, device=dev, dtype=torch.bfloat16)
        i = [0]

        def fn():
            w = ws[i[0] % copies]
            i[0] += 1
            if a.kernel == "gemm_library":
                torch.mm(x[:a.m], w.t(), out=y[:a.m])
            elif a.kernel.startswith("gemm_skinny"):
                ops.gemm_bf16_skinny_tcgen05(x, w, y, a.m, swiglu=swiglu)
            elif a.kernel.startswith("gemm_tc"):
                ops.gemm_bf16_tcgen05(x, w, y, a.m, swiglu=swiglu, pair=not a.kernel.startswith("gemm_tc1"))
            else:
                ops.gemm_bf16_smallm(x, w, y, a.m, swiglu=swiglu)
        timed(fn, wbytes, 2.0 * a.m * rows * a.k)
        return 0

    if a.kernel == "attention_decode":
        from .parts.attention import decode_plan
        hd, kvh, qh, B, ctx = a.head_dim, a.kv_heads, a.q_heads, a.batch, a.context
        pages_per = (ctx + 63) // 64
        kv_bytes = B * pages_per * 2 * kvh * 64 * hd * 2
        copies = max(2, int(math.ceil(256e6 / kv_bytes)) + 1)
        n_pages = B * pages_per
        stores = [torch.randn(n_pages, 2, kvh, 64, hd, device=dev).bfloat16() for _ in range(copies)]
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(B, pages_per).contiguous()
        views = [ops.PagedCacheArg(s.data_ptr(), table.data_ptr(), 2 * kvh * 64 * hd, pages_per, pages_per, 64, kvh, hd,
                                   n_pages) for s in stores]
        q = torch.randn(B, qh * hd, device=dev).bfloat16()
        out = torch.empty_like(q)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)

        class Ctx:
            max_context = ctx
            sm_count = torch.cuda.get_device_properties(0).multi_processor_count
        splits, groups = (a.splits, max(1, a.groups)) if a.splits else decode_plan(Ctx, B, kvh, qh, hd)
        scratch = torch.zeros(max(1, ops.attention_decode_scratch_bytes(B, qh, kvh, hd, splits)), dtype=torch.uint8,
                              device=dev)
        i = [0]

        def fn():
            v = views[i[0] % copies]
            i[0] += 1
            ops.attention_decode_bf16(q, out, v, slots, pos, B, qh, 1 / math.sqrt(hd), 0, splits,
                                      scratch if (groups > 1 or a.scratch_merge or splits > ops.ATTENTION_DECODE_CLUSTER_SPLITS)
                                      else None, groups=groups)
        print(f"splits {splits} in {groups} cluster(s)", file=sys.stderr)
        timed(fn, B * ctx * 2 * kvh * hd * 2, 4.0 * B * qh * hd * ctx)
        return 0

    if a.kernel in ("attention_prefill", "attention_prefill_tc"):
        hd, kvh, qh, T = a.head_dim, a.kv_heads, a.q_heads, a.context
        pages_per = (T + 63) // 64
        store = torch.randn(pages_per, 2, kvh, 64, hd, device=dev).bfloat16()
        table = torch.arange(pages_per, dtype=torch.int32, device=dev).reshape(1, pages_per).contiguous()
        view = ops.PagedCacheArg(store.data_ptr(), table.data_ptr(), 2 * kvh * 64 * hd, pages_per, pages_per, 64, kvh,
                                 hd, pages_per)
        q = torch.randn(T, qh * hd, device=dev).bfloat16()
        out = torch.empty_like(q)
        mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)   # noqa: E731
        tr = ops.attention_prefill_tile_rows()
        n_tiles = (T + tr - 1) // tr
        tile_seq, tile_row0 = mk([0] * n_tiles), mk(list(range(0, T, tr)))
        first, sslot, spos0 = mk([0, T]), mk([0]), mk([0])
        copies = 1

        def fn():
            if a.kernel == "attention_prefill_tc":
                ops.attention_prefill_tcgen05(q, out, view, tile_seq, tile_row0, n_tiles, first, sslot, spos0, qh,
                                              1 / math.sqrt(hd), 0)
            else:
                ops.attention_prefill_bf16(q, out, view, tile_seq, tile_row0, n_tiles, first, sslot, spos0, qh,
                                           1 / math.sqrt(hd), 0)
        timed(fn, 2 * T * qh * hd * 2 + 2 * T * kvh * hd * 2, 4.0 * qh * hd * T * (T + 1) / 2)
        return 0

    if a.kernel == "add_rmsnorm":
        rows, h = a.m, a.n
        resid = torch.randn(rows, h, device=dev)
        delta = torch.randn(rows, h, device=dev).bfloat16()
        w = torch.ones(h, device=dev)
        out = torch.empty_like(delta)
        copies = 1
        timed(lambda: ops.add_rmsnorm(resid, delta, w, out, rows, 1e-6), rows * h * (4 + 4 + 2 + 2))
        return 0
    if a.kernel == "swiglu":
        rows, inter = a.m, a.n
        gu = torch.randn(rows, 2 * inter, device=dev).bfloat16()
        out = torch.empty(rows, inter, device=dev, dtype=torch.bfloat16)
        copies = 1
        timed(lambda: ops.swiglu(gu, out, rows), rows * inter * 6)
        return 0
    if a.kernel == "qk_norm_rope":
        # a.m rows of one sequence at positions 0 .. m-1: q/k head norm, rotation from the table, K/V into the pages
        hd, kvh, qh, rows = a.head_dim, a.kv_heads, a.q_heads, a.m
        pages_per = (rows + 63) // 64
        store = torch.zeros(pages_per, 2, kvh, 64, hd, device=dev, dtype=torch.bfloat16)
        table = torch.arange(pages_per, dtype=torch.int32, device=dev).reshape(1, pages_per).contiguous()
        view = ops.PagedCacheArg(store.data_ptr(), table.data_ptr(), 2 * kvh * 64 * hd, pages_per, pages_per, 64, kvh,
                                 hd, pages_per)
        qkv = torch.randn(rows, (qh + 2 * kvh) * hd, device=dev).bfloat16()
        q_out = torch.empty(rows, qh * hd, device=dev, dtype=torch.bfloat16)
        ones = torch.ones(hd, device=dev)
        inv_freq = (1e6 ** (-torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd)).contiguous()
        ang = torch.arange(rows, device=dev, dtype=torch.float32)[:, None] * inv_freq[None, :]
        rope_table = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous()
        slot = torch.zeros(rows, dtype=torch.int32, device=dev)
        pos = torch.arange(rows, dtype=torch.int32, device=dev)
        copies = 1
        moved = rows * ((qh + 2 * kvh) * hd * 2 + qh * hd * 2 + 2 * kvh * hd * 2)
        timed(lambda: ops.qk_norm_rope_kv_write(qkv, ones, ones, inv_freq, hd, q_out, view, slot, pos, rows, qh, 1e-6,
                                                True, rope_table), moved)
        return 0
    print(f"unknown kernel {a.kernel!r}", file=sys.stderr)
    return 2


def _kernel_bench_reference(a, timed) -> int:
    """The reference project's kernel of the asked name at the asked sizes (one sequence), from its
    unmodified sources; inputs of the same shapes and distributions as this library's case, in the
    reference's own layouts (contiguous cache [max_ctx][kv_heads][128], bfloat16 norm weights)."""
    import math
    import torch
    from . import reference_kernels as R
    dev = "cuda:0"
    try:
        k = R.load()
    except R.ReferenceUnavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e).splitlines()[0]}))
        return 0
    hd, kvh, qh = a.head_dim, a.kv_heads, a.q_heads
    if hd != R.HEAD_DIM:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's kernels are written for head size {R.HEAD_DIM}"}))
        return 0
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    u32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)   # noqa: E731
    bf = lambda *shape: torch.randn(*shape, device=dev).bfloat16()     # noqa: E731
    if a.kernel == "decode_step":
        # the reference's kernels and cuBLAS in the reference engine's order, one sequence, as a CUDA graph
        step = R.DecodeStepInReferenceOrder(k, a.layers, a.n, a.k, qh, kvh, a.vocab, a.context)
        for _ in range(3):
            step.launch()
        step.reset()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step.launch()
        steps = min(a.iters, 60)
        step.reset()
        g.replay()
        step.reset()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(steps):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / steps
        bytes_step = step.weight_bytes() + a.layers * 2 * (a.context + steps / 2) * kvh * hd * 2
        print(json.dumps({"kernel": "decode_step", "impl": "reference kernels + cuBLAS in the reference engine's order, launched by this "
                          "library's host code (not the reference engine)", "layers": a.layers, "hidden": a.n, "intermediate": a.k,
                          "context": a.context, "batch": 1, "ms_per_step": ms, "tokens_per_s": 1e3 / ms,
                          "gb_s": bytes_step / ms / 1e6, "token_after": int(step.token[0])}))
        return 0
    if a.kernel == "attention_decode":
        ctx = a.context
        kv_bytes = 2 * ctx * kvh * hd * 2
        copies = max(2, int(math.ceil(256e6 / kv_bytes)) + 1)
        caches = [(bf(ctx, kvh, hd), bf(ctx, kvh, hd)) for _ in range(copies)]
        q, out, pos = bf(1, qh * hd), torch.empty(1, qh * hd, device=dev, dtype=torch.bfloat16), u32(ctx - 1)
        plan = R.split_plan(k, qh, kvh, sms)
        state = torch.zeros(qh * plan[2] * R.SPLIT_STATE, device=dev)
        counter = torch.zeros(max(kvh, qh), dtype=torch.int32, device=dev)
        print(f"reference split plan: kernel {plan[0]}, grid {plan[1]} x {plan[2]}", file=sys.stderr)
        i = [0]

        def fn():
            kc, vc = caches[i[0] % copies]
            i[0] += 1
            R.attention_decode(k, q, kc, vc, state, counter, out, pos, qh, kvh, ctx, 1 / math.sqrt(hd), plan)
        timed(fn, kv_bytes, 4.0 * qh * hd * ctx, copies)
        return 0
    if a.kernel == "attention_prefill":
        T = a.context
        kc, vc, q = bf(T, kvh, hd), bf(T, kvh, hd), bf(T, qh * hd)
        out, pos0 = torch.empty_like(q), u32(0)
        timed(lambda: R.attention_prefill(k, q, kc, vc, out, pos0, T, qh, kvh, T, 1 / math.sqrt(hd)),
              2 * T * qh * hd * 2 + 2 * T * kvh * hd * 2, 4.0 * qh * hd * T * (T + 1) / 2, 1)
        return 0
    if a.kernel == "add_rmsnorm":
        rows, h = a.m, a.n
        resid, delta, w = torch.randn(rows, h, device=dev), bf(rows, h), torch.ones(h, device=dev).bfloat16()
        out = torch.empty_like(delta)
        timed(lambda: R.add_rmsnorm(k, resid, delta, w, out, rows, h, 1e-6), rows * h * (4 + 4 + 2 + 2), 0.0, 1)
        return 0
    if a.kernel == "qk_norm_rope":
        rows = a.m
        qkv, q_out = bf(rows, (qh + 2 * kvh) * hd), torch.empty(rows, qh * hd, device=dev, dtype=torch.bfloat16)
        kc, vc = torch.zeros(rows, kvh, hd, device=dev, dtype=torch.bfloat16), torch.zeros(rows, kvh, hd, device=dev, dtype=torch.bfloat16)
        ones = torch.ones(hd, device=dev).bfloat16()
        inv_freq = (1e6 ** (-torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd)).contiguous()
        pos0 = u32(0)
        moved = rows * ((qh + 2 * kvh) * hd * 2 + qh * hd * 2 + 2 * kvh * hd * 2)
        timed(lambda: R.qk_norm_rope_kv_write(k, qkv, ones, ones, inv_freq, q_out, kc, vc, pos0, rows, qh, kvh, rows, 1e-6),
              moved, 0.0, 1)
        return 0
    if a.kernel == "swiglu":
        rows, inter = a.m, a.n
        gu, out = bf(rows, 2 * inter), torch.empty(rows, inter, device=dev, dtype=torch.bfloat16)
        timed(lambda: R.swiglu(k, gu, out, rows, inter), rows * inter * 6, 0.0, 1)
        return 0
    print(json.dumps({"impl": "reference", "unavailable": f"the reference has no kernel for {a.kernel!r}"}))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        return cmd_replay(None, argv[1:])
    ap = argparse.ArgumentParser(prog="x0ne_engine_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate")
    g.add_argument("model")
    g.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat per prompt")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--stop-token-ids", default=None)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--decode", default="graph", choices=["graph", "eager"])
    g.add_argument("--max-ctx", type=int, default=None)
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("core-bench")
    b.add_argument("model")
    b.add_argument("--lengths", default="short,1k,4k")
    b.add_argument("--decode", type=int, default=256)
    b.add_argument("--reps", type=int, default=5)
    b.add_argument("--batch", type=int, default=1)
    b.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    b.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="random weights made on the device from config.json alone (no safetensors needed)")
    b.add_argument("--clock-trace", action="store_true",
                   help="read the SM clock (NVML) every millisecond during the last repetition and report the "
                        "stretches of one clock value with the token gaps that fell into each")
    b.set_defaults(fn=cmd_core_bench)

    t = sub.add_parser("step-timeline")
    t.add_argument("model")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=3072)
    t.add_argument("--random-weights", type=int, default=None, metavar="SEED")
    t.set_defaults(fn=cmd_step_timeline)

    r = sub.add_parser("roofline")
    r.add_argument("--config", required=True)
    r.add_argument("--gpu", type=float, required=True, help="memory bandwidth in GB/s")
    r.add_argument("--prompt", type=int, required=True)
    r.add_argument("--generated", type=int, required=True)
    r.add_argument("--tok-s", type=float, default=None)
    r.add_argument("--batch", type=int, default=1)
    r.set_defaults(fn=cmd_roofline)

    i = sub.add_parser("init")
    i.add_argument("config")
    i.add_argument("out")
    i.add_argument("--seed", type=int, default=0)
    i.add_argument("--linear-std", type=float, default=0.02)
    i.add_argument("--norm-jitter", type=float, default=0.0)
    i.set_defaults(fn=cmd_init)

    k = sub.add_parser("kernel-bench")
    k.add_argument("--kernel", required=True)
    k.add_argument("--impl", default="ours", choices=["ours", "reference"])
    k.add_argument("--m", type=int, default=8)
    k.add_argument("--n", type=int, default=4096)
    k.add_argument("--k", type=int, default=4096)
    k.add_argument("--batch", type=int, default=8)
    k.add_argument("--context", type=int, default=3072)
    k.add_argument("--scratch-merge", action="store_true",
                   help="attention_decode: merge the splits through global scratch even where a cluster could")
    k.add_argument("--q-heads", type=int, default=32)
    k.add_argument("--kv-heads", type=int, default=8)
    k.add_argument("--head-dim", type=int, default=128)
    k.add_argument("--splits", type=int, default=0)
    k.add_argument("--groups", type=int, default=1,
                   help="attention_decode: with --splits, how many thread-block clusters the splits of a (sequence, kv head) form")
    k.add_argument("--layers", type=int, default=36, help="decode_step (--impl reference): layers of the model")
    k.add_argument("--vocab", type=int, default=151936, help="decode_step (--impl reference): vocabulary")
    k.add_argument("--iters", type=int, default=50)
    k.add_argument("--warmup", type=int, default=5)
    k.set_defaults(fn=cmd_kernel_bench)

    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
