"""The choice of how many blocks a decode attention launch gives each (sequence, kv head): host
arithmetic only, with the GPU's answers (how many clusters of a size run at once) stubbed."""
import pytest

from x0ne_engine_b200.csrc import ops
from x0ne_engine_b200.parts import attention

FIT = {1: 296, 2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33}      # a B200 at head_dim 128


class Ctx:
    sm_count = 148

    def __init__(self, max_context):
        self.max_context = max_context


@pytest.fixture
def stub(monkeypatch):
    monkeypatch.setattr(ops, "attention_decode_max_clusters", lambda hd, s: FIT.get(s, 0))
    monkeypatch.setattr(ops, "attention_decode_blocks_per_sm", lambda: 2)


def splits(batch, ctx=4096, kv_heads=8, q_heads=32):
    return attention.decode_splits(Ctx(ctx), batch, kv_heads, q_heads, 128)


def test_a_small_batch_is_split_until_it_fills_the_gpu_once(stub):
    assert splits(1) == 8 and splits(4) == 8             # 8 and 32 units: clusters of 8 (33 fit)
    assert splits(8) == 4                                 # 64 units: 71 clusters of 4 fit, 56 of 5 do not
    assert splits(9) == 3 and splits(16) == 2             # 72 and 128 units
    for b in (1, 2, 4, 8, 9, 16):
        s = splits(b)
        assert b * 8 <= FIT[s]                            # one wave


def test_a_batch_past_one_wave_is_split_where_that_shortens_the_waves(stub):
    assert splits(32) == 1                                # 256 blocks: one wave as they are
    assert splits(48) == 2                                # 384 blocks: 2 waves whole, 3 waves of halves
    assert splits(64) == 1                                # 512 blocks: 2 waves either way


def plan(batch, ctx, kv_heads=8, q_heads=32):
    return attention.decode_plan(Ctx(ctx), batch, kv_heads, q_heads, 128)


def test_no_more_splits_than_pages_or_than_the_kernel_takes(stub):
    assert splits(1, ctx=64) == 1 and splits(1, ctx=130) <= 3
    for b in range(1, 70):
        s, g = plan(b, 1 << 20)
        assert s <= ops.ATTENTION_DECODE_MAX_SPLITS and s % g == 0
        assert s // g <= ops.ATTENTION_DECODE_CLUSTER_SPLITS and (g == 1 or s // g >= 2)


def test_one_or_two_long_sequences_get_several_clusters_per_kv_head(stub):
    """64 blocks cannot draw the memory's bandwidth; measured on a B200, four clusters of 8 take
    30.5 us instead of 57.4 at 32,768 keys, 13.3 instead of 15.0 at 6,144, 12.4 instead of 11.7 at 4,096."""
    assert plan(1, 4096) == (8, 1) and plan(2, 4096) == (8, 1)        # short: the meeting in scratch costs what it saves
    assert plan(1, 6144) == (32, 4) and plan(1, 8192) == (32, 4) and plan(1, 32768) == (32, 4)
    assert plan(2, 6144) == (16, 4) and plan(2, 8192) == (16, 4) and plan(2, 32768) == (16, 4)
    for ctx in (8192, 32768, 1 << 17):
        assert plan(4, ctx) == (8, 1)                                 # 256 blocks already: nothing to gain
        for b in (1, 2, 3, 4):
            s, g = plan(b, ctx)
            assert b * 8 * g <= FIT[s // g]                           # all clusters run at once
    # the scratch the mixer asks its workspace for covers every launch of that kind
    need = attention.decode_scratch_bytes(Ctx(32768), 8, 32, 128)
    for b in (1, 2, 3, 4):
        s, g = plan(b, 32768)
        if g > 1:
            rows_parts = b * 32 * g
            assert need >= rows_parts * 128 * 4 + rows_parts * 8 + 256


def test_unknown_capacity_falls_back_to_a_margin(monkeypatch):
    monkeypatch.setattr(ops, "attention_decode_max_clusters", lambda hd, s: 0)
    monkeypatch.setattr(ops, "attention_decode_blocks_per_sm", lambda: 2)
    s = splits(8)
    assert 1 <= s <= 8 and 64 * s <= 296
