"""The manifest that trace replay keeps beside its logits files: written, read back and checked."""
import hashlib
import json
import os

import numpy as np
import pytest

from x0ne_engine_b200.engine.replay import MANIFEST, check_manifest, write_manifest


def _record(out, step, rows, vocab, seed):
    data = np.random.default_rng(seed).standard_normal((rows, vocab)).astype("<f4").tobytes()
    with open(os.path.join(out, f"{step}.f32"), "wb") as f:
        f.write(data)
    return {"file": f"{step}.f32", "step": step, "shape": [rows, vocab], "dtype": "float32-le",
            "sha256": hashlib.sha256(data).hexdigest()}


def test_manifest_round_trip_and_every_way_a_file_can_be_wrong(tmp_path):
    out = str(tmp_path)
    head = {"schema": 1, "model": "/m", "architecture": "X", "dtype": "float32", "vocab_size": 7}
    files = [_record(out, 0, 3, 7, 1), _record(out, 4, 1, 7, 2)]
    write_manifest(out, head, files)
    man = check_manifest(out)
    assert man["vocab_size"] == 7 and [f["step"] for f in man["files"]] == [0, 4]
    assert not os.path.exists(os.path.join(out, MANIFEST + ".tmp"))

    with open(os.path.join(out, "0.f32"), "r+b") as f:          # one flipped byte
        f.seek(5)
        b = f.read(1)
        f.seek(5)
        f.write(bytes([b[0] ^ 1]))
    with pytest.raises(ValueError, match=r"0\.f32: the bytes do not have the recorded SHA-256"):
        check_manifest(out)

    files[0] = _record(out, 0, 3, 7, 1)
    with open(os.path.join(out, "4.f32"), "ab") as f:           # a file longer than its shape
        f.write(b"\0\0\0\0")
    write_manifest(out, head, files)
    with pytest.raises(ValueError, match=r"4\.f32: 32 bytes, the manifest's shape \[1, 7\] gives 28"):
        check_manifest(out)

    os.remove(os.path.join(out, "4.f32"))                       # a file that is gone
    with pytest.raises(ValueError, match=r"4\.f32"):
        check_manifest(out)
    with open(os.path.join(out, MANIFEST)) as f:
        assert json.load(f)["files"][1]["file"] == "4.f32"
