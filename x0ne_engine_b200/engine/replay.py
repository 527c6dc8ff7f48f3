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

Beside the logits files the run keeps `<out>/manifest.json`: for every file its name, its shape
[wanted, vocab], its dtype and the SHA-256 of its bytes, with the model folder, the dtype of the run
and the vocabulary, rewritten (through a temporary file) after every step that wrote logits, so a
reader can check a file before it trusts it.  The library engine pairs its reference logits with
the same facts (x0ne-core/runtime/src/refs.rs:17-42,112-153); `check_manifest` is the reader's side.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Dict, List

MANIFEST = "manifest.json"


def write_manifest(out_dir: str, head: dict, files: List[dict]) -> None:
    tmp = os.path.join(out_dir, MANIFEST + ".tmp")
    with open(tmp, "w") as f:
        json.dump({**head, "files": files}, f, indent=1)
    os.replace(tmp, os.path.join(out_dir, MANIFEST))


def check_manifest(out_dir: str) -> dict:
    """Reads `<out_dir>/manifest.json` and checks every listed file: present, of the length its
    shape gives, with the recorded SHA-256.  Returns the manifest; raises ValueError with every
    difference otherwise."""
    with open(os.path.join(out_dir, MANIFEST)) as f:
        man = json.load(f)
    bad = []
    for rec in man.get("files", []):
        path = os.path.join(out_dir, rec["file"])
        try:
            with open(path, "rb") as f:
                data = f.read()
        except OSError as e:
            bad.append(f"{rec['file']}: {e}")
            continue
        want_len = 4 * rec["shape"][0] * rec["shape"][1]
        if rec.get("dtype") != "float32-le" or len(data) != want_len:
            bad.append(f"{rec['file']}: {len(data)} bytes, the manifest's shape {rec['shape']} gives {want_len}")
        elif hashlib.sha256(data).hexdigest() != rec["sha256"]:
            bad.append(f"{rec['file']}: the bytes do not have the recorded SHA-256")
    if bad:
        raise ValueError("the logits files do not match their manifest:\n  " + "\n  ".join(bad))
    return man



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--max-step-tokens", type=int, default=None,
                    help="most rows the engine runs in one pass; a larger step is cut into several passes "
                         "(default: the cache's capacity, at most 4096)")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    if args.max_step_tokens is not None and args.max_step_tokens <= 0:
        ap.error("--max-step-tokens must be positive")

    print("[x0ne-b200] trace_run: loading (kernels are compiled at the first call of a fresh checkout)",
          file=sys.stderr, flush=True)
    from .engine import Engine
    from ..cache import PAGE_SIZE, pages_for

    os.makedirs(args.out, exist_ok=True)
    capacity = pages_for(args.max_tokens, PAGE_SIZE) * PAGE_SIZE
    engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device, max_tokens=capacity,
                                max_step_tokens=args.max_step_tokens or min(capacity, 4096))
    print(f"[x0ne-b200] trace_run: {engine.describe()}", file=sys.stderr, flush=True)
    head = {"schema": 1, "model": os.path.abspath(args.model), "architecture": engine.spec.architecture,
            "dtype": args.dtype, "vocab_size": engine.vocab_size, "max_tokens": capacity,
            "max_step_tokens": engine.max_step_tokens}
    files: List[dict] = []
    write_manifest(args.out, head, files)
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
                data = logits.detach().to("cpu").numpy().astype("<f4", copy=False).tobytes()
                name = f"{step}.f32"
                with open(os.path.join(args.out, name), "wb") as f:
                    f.write(data)
                files.append({"file": name, "step": step, "shape": [int(logits.shape[0]), int(logits.shape[1])],
                              "dtype": "float32-le", "sha256": hashlib.sha256(data).hexdigest()})
                write_manifest(args.out, head, files)
        for rid in rec.get("end", []):
            slot = slots.pop(str(rid), None)
            if slot is not None:
                engine.free_sequence(slot)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
