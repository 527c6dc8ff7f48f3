#!/usr/bin/env python3
"""Copies the tiny float32 Qwen3 checkpoint that x0ne-labs/x0ne-Engine keeps for its own
decoder tests, with the outputs its upstream implementation gave, into tests/golden/qwen3_f32.

usage: make_golden.py <root of an x0ne-Engine checkout>

Source: x0ne-infer/tests/arch/qwen3/{config.json, model.safetensors, reference.json}, written
by x0ne-infer/scripts/make-arch-fixtures.py:110-183 (float32, eager attention, seed 1234, init
range 0.5, norm weights 1 + 0.2 randn).  Kept from reference.json: the 12 ids, logits [12, 40],
per-layer hidden states [4][12, 24], per-layer attention probabilities [4][3, 12, 12], the
6-token prompt and the 10 greedy tokens.  The project's Rust model code cannot be built without
a Rust toolchain, so this data, not a call into that code, is what the plain implementation
in tests/plain_impl.py is checked against.
"""
import json
import os
import shutil
import sys

KEEP = ["ids", "logits", "hidden", "attentions", "prompt", "generated"]


def main():
    src = os.path.join(sys.argv[1], "x0ne-infer", "tests", "arch", "qwen3")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qwen3_f32")
    os.makedirs(dst, exist_ok=True)
    for name in ("config.json", "model.safetensors"):
        shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
    with open(os.path.join(src, "reference.json")) as f:
        ref = json.load(f)
    with open(os.path.join(dst, "reference.json"), "w") as f:
        json.dump({k: ref[k] for k in KEEP}, f)


if __name__ == "__main__":
    main()
