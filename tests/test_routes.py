"""The routing table of the bfloat16 products: what it chooses at the matrices of the three model
sizes it was measured at, and that every row count of every shape gets an answer."""
import pytest

from x0ne_engine_b200.csrc import routes

# hidden, intermediate, q heads, kv heads (head size 128)
SIZES = {"1.7B": (2048, 6144, 16, 8), "8B": (4096, 12288, 32, 8), "32B": (5120, 25600, 64, 8)}


def matrices(size):
    h, inter, qh, kvh = SIZES[size]
    return dict(qkv=((qh + 2 * kvh) * 128, h), o=(h, qh * 128), down=(h, inter), gate_up=(2 * inter, h))


@pytest.mark.parametrize("size,rows,expect", [
    ("8B", 1, dict(qkv="smallm", o="smallm", down="smallm", gate_up="smallm")),
    ("8B", 8, dict(qkv="smallm", o="smallm", down="smallm", gate_up="smallm")),
    ("8B", 16, dict(qkv="skinny", o="skinny", down="skinny", gate_up="skinny")),
    ("8B", 64, dict(qkv="library", o="library", down="skinny", gate_up="skinny")),
    ("8B", 128, dict(qkv="library", o="library", down="library", gate_up="library")),
    ("8B", 2048, dict(qkv="library", o="library", down="library", gate_up="tc_pair")),
    ("1.7B", 8, dict(qkv="smallm", o="smallm", down="smallm", gate_up="smallm")),
    ("1.7B", 16, dict(qkv="smallm", o="smallm", down="skinny", gate_up="smallm")),
    ("1.7B", 32, dict(qkv="library", o="library", down="skinny", gate_up="skinny")),
    ("32B", 1, dict(qkv="smallm", o="library", down="library", gate_up="smallm")),
    ("32B", 8, dict(qkv="smallm", o="library", down="library", gate_up="smallm")),
    ("32B", 32, dict(qkv="skinny", o="skinny", down="skinny", gate_up="skinny")),
    ("32B", 64, dict(qkv="library", o="library", down="skinny", gate_up="skinny")),
])
def test_choices_at_the_measured_sizes(size, rows, expect):
    got = {name: routes.kernel_for(rows, n, k, fused=name == "gate_up") for name, (n, k) in matrices(size).items()}
    assert got == expect


def test_every_row_count_of_every_shape_has_a_rule_and_every_rule_is_reached():
    reached = set()
    shapes = [(n, k) for size in SIZES for n, k in matrices(size).values()] + [(64, 64), (160, 96), (151936, 4096), (8, 8)]
    for n, k in shapes:
        for fused in (False, True):
            for rows in list(range(1, 130)) + [767, 768, 5000, 1 << 20]:
                rule = routes.choose(rows, n, k, fused=fused)
                assert rule.kernel in ("smallm", "skinny", "tc_pair", "library") and rule.why
                reached.add(id(rule))
    assert len(reached) == len(routes.RULES)
    assert routes.RULES[-1].kernel == "library" and routes.RULES[-1].rows == (1, 1 << 30) and routes.RULES[-1].fused is None


def test_fill_of_the_weight_streaming_kernel():
    assert routes.Shape(4096, 4096).smallm_fill == pytest.approx(256 / 296)          # one tile each on 256 of 296 blocks
    assert routes.Shape(6144, 4096).smallm_fill == pytest.approx(192 / 296)          # two tiles each on 192
    assert routes.Shape(5120, 25600).smallm_fill == pytest.approx(160 / 296)
    assert routes.Shape(5120, 25600).long_rows and not routes.Shape(6144, 4096).long_rows
