"""The row counts that short prompt passes are launched with."""
from x0ne_engine_b200.engine.engine import PASS_GRAPH_MAX_ROWS, padded_rows


def test_padded_rows_are_few_and_never_fewer_than_the_rows():
    seen = set()
    for n in range(1, PASS_GRAPH_MAX_ROWS + 1):
        p = padded_rows(n)
        assert p >= n and p - n < 64
        assert padded_rows(p) == p
        if n > 1:
            assert p >= padded_rows(n - 1)
        seen.add(p)
    assert len(seen) == 8 + 4 + (PASS_GRAPH_MAX_ROWS - 64) // 64
    assert [padded_rows(n) for n in (1, 8, 9, 16, 17, 64, 65, 128, 129)] == [1, 8, 16, 16, 32, 64, 128, 128, 192]
