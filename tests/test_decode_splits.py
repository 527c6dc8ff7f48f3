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


def test_no_more_splits_than_pages_or_than_a_cluster_holds(stub):
    assert splits(1, ctx=64) == 1 and splits(1, ctx=130) <= 3
    assert max(splits(b, ctx=1 << 20) for b in range(1, 70)) <= ops.ATTENTION_DECODE_CLUSTER_SPLITS


def test_unknown_capacity_falls_back_to_a_margin(monkeypatch):
    monkeypatch.setattr(ops, "attention_decode_max_clusters", lambda hd, s: 0)
    monkeypatch.setattr(ops, "attention_decode_blocks_per_sm", lambda: 2)
    s = splits(8)
    assert 1 <= s <= 8 and 64 * s <= 296
