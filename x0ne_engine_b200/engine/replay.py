"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: every step is one call
of `Engine.step`, the function generation uses.  In the library engine the counterpart is the
teacher-forced `Engine::run` / `logits_at` (x0ne-core/runtime/src/engine.rs:929-1016).

Input, one JSON object a line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` gives each request's next tokens and the places among them whose logits are wanted;
`end` names requests that are finished after the step, whose cache is given back.  For a step
that wants something, `<out>/<step>.f32` receives the logits [wanted, vocab] as little-endian
float32 in the order of the entries and of `want`.  After every step the line `done <step>` is
printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")

    print("[x0ne-b200] trace_run: loading (kernels are compiled at the first call of a fresh checkout)",
          file=sys.stderr, flush=True)
    from .engine import Engine
    from ..cache import PAGE_SIZE, pages_for

    os.makedirs(args.out, exist_ok=True)
    capacity = pages_for(args.max_tokens, PAGE_SIZE) * PAGE_SIZE
    engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device, max_tokens=capacity,
                                max_step_tokens=min(capacity, 4096))
    print(f"[x0ne-b200] trace_run: {engine.describe()}", file=sys.stderr, flush=True)
    slots: Dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        ids = [str(e["id"]) for e in entries]
        for rid in ids:
            if rid not in slots:
                slots[rid] = engine.new_sequence()
        if entries:
            logits = engine.step([slots[r] for r in ids], [e["tokens"] for e in entries],
                                 [e.get("want", []) for e in entries])
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            slot = slots.pop(str(rid), None)
            if slot is not None:
                engine.free_sequence(slot)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
