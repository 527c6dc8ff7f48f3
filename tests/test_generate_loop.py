"""The generation loop's decisions on the CPU, with a scripted runner in place of the GPU."""
import pytest

from x0ne_engine_b200.engine.generate import (FINISHED_PICK, NAN_PICK, GenerationError, Generator, Row, plan_batches,
                                              run_batch)
from x0ne_engine_b200.sampling import PromptTooLong, SamplingParams, generation_budget


class Scripted:
    """Each request's picks are scripted; records what the loop asks for."""

    def __init__(self, scripts):
        self.scripts = scripts            # request index -> list of picks
        self.log = []
        self.at = {}
        self.open = False
        self.rows = None

    def start(self, rows):
        assert not self.open
        self.open, self.rows = True, rows
        self.log.append(("start", [r.request for r in rows]))
        out = []
        for r in rows:
            self.at[r.request] = 1
            out.append(self.scripts[r.request][0])
        return out

    def step(self, live):
        self.log.append(("step", [self.rows[i].request for i in live]))
        out = []
        for i in live:
            req = self.rows[i].request
            out.append(self.scripts[req][self.at[req]])
            self.at[req] += 1
        return out

    def close(self):
        self.open = False
        self.log.append(("close",))


class FakeEngine:
    max_seq_len = 32
    vocab_size = 100

    class cache:
        page_size = 64

        @staticmethod
        def free_tokens():
            return 64 * 3


def gen(scripts, prompts, params, max_batch=2):
    runner = Scripted(scripts)
    g = Generator(FakeEngine(), max_batch=max_batch, runner_factory=lambda: runner)
    return g.generate(prompts, params), runner


def test_budget():
    assert generation_budget(10, 50, 32) == 22 and generation_budget(10, 5, 32) == 5
    with pytest.raises(PromptTooLong):
        generation_budget(32, 5, 32)


def test_stop_token_is_not_emitted_fed_or_counted_and_rows_leave_early():
    scripts = {0: [5, 6, 99, 1, 1], 1: [7, 8, 9, 10, 11], 2: [99]}
    p = SamplingParams(max_tokens=4, stop_token_ids=(99,))
    out, runner = gen(scripts, [[1, 2], [3], [4, 4, 4]], p)
    assert [c.tokens for c in out] == [[5, 6], [7, 8, 9, 10], []]
    assert [c.finish_reason for c in out] == ["stop", "length", "stop"]
    assert [c.prompt_tokens for c in out] == [2, 1, 3]
    # batch 1 holds requests 0 and 1; request 0 leaves after its stop; the last token of a budget is not fed
    assert runner.log == [("start", [0, 1]), ("step", [0, 1]), ("step", [0, 1]), ("step", [1]), ("close",),
                          ("start", [2]), ("close",)]


def test_budget_is_cut_by_the_context_and_a_full_prompt_is_refused():
    scripts = {0: list(range(40))}
    out, _ = gen(scripts, [[1] * 30], SamplingParams(max_tokens=10))
    assert out[0].tokens == [0, 1] and out[0].finish_reason == "length"
    with pytest.raises(PromptTooLong):
        gen(scripts, [[1] * 32], SamplingParams(max_tokens=10))


def test_bad_requests_are_refused_before_anything_runs():
    for prompts in ([[]], [[100]], [[-1]]):
        with pytest.raises(ValueError):
            gen({0: [1]}, prompts, SamplingParams())
    with pytest.raises(ValueError, match="top_k"):
        SamplingParams.from_options(top_k=5)
    with pytest.raises(ValueError, match="unknown"):
        SamplingParams.from_options(beam=5)
    for bad in (dict(max_tokens=0), dict(temperature=-1.0), dict(top_p=float("nan")), dict(seed=-1)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_nan_pick_fails_the_request_and_the_batch_is_closed():
    runner = Scripted({0: [3, NAN_PICK]})
    rows = [Row(0, [1], SamplingParams(max_tokens=5), 5, 0)]
    with pytest.raises(GenerationError, match="NaN"):
        run_batch(runner, rows)
    assert runner.log[-1] == ("close",)
    runner = Scripted({0: [FINISHED_PICK]})
    with pytest.raises(GenerationError):
        run_batch(runner, [Row(0, [1], SamplingParams(max_tokens=5), 5, 0)])


def test_plan_batches_respects_batch_size_and_cache_room():
    assert plan_batches([10, 10, 10, 10, 10], 2, 10_000, 64) == [(0, 2), (2, 4), (4, 5)]
    assert plan_batches([100, 30, 64, 65], 8, 192, 64) == [(0, 2), (2, 4)]
    assert plan_batches([100, 30, 65, 65], 8, 192, 64) == [(0, 2), (2, 3), (3, 4)]
    with pytest.raises(GenerationError):
        plan_batches([300], 8, 192, 64)


def test_greedy_reading_of_the_options():
    assert SamplingParams().greedy and SamplingParams(temperature=1e-8).greedy
    assert SamplingParams(temperature=0.7, top_p=0.0).greedy and not SamplingParams(temperature=0.7).greedy


def test_each_request_gets_its_own_params_and_seed():
    scripts = {0: [1, 2, 3], 1: [4, 5, 6]}
    params = [SamplingParams(max_tokens=1, seed=3), SamplingParams(max_tokens=3, temperature=0.5)]
    runner = Scripted(scripts)
    g = Generator(FakeEngine(), max_batch=4, runner_factory=lambda: runner)
    out = g.generate([[1], [2]], params)
    assert [len(c.tokens) for c in out] == [1, 3]
    assert runner.rows[0].seed == 3 and 0 <= runner.rows[1].seed < 1 << 53


def test_token_gaps_are_stamped_per_step_and_summarised():
    """One host timestamp per decode step: the gaps between them (the first from the prompts' picks)
    are kept, and decode time runs to the last token's arrival."""
    from x0ne_engine_b200.engine.generate import GenerationStats, percentiles
    ticks = iter([0.0, 1.0, 1.5, 1.75, 4.0, 9.0])
    rows = [Row(0, [1], SamplingParams(max_tokens=4), 4, 0), Row(1, [2], SamplingParams(max_tokens=2), 2, 0)]
    stats = GenerationStats()
    run_batch(Scripted({0: [5, 6, 7, 8], 1: [5, 6]}), rows, stats, clock=lambda: next(ticks))
    assert stats.token_gaps == [0.5, 0.25, 2.25] and stats.decode_steps == 3 and stats.decode_tokens == 2 + 1 + 1
    assert stats.prefill_seconds == 1.0 and stats.decode_seconds == 3.0
    assert stats.gap_percentiles() == {"p50": 0.5, "p90": 2.25, "p99": 2.25, "max": 2.25, "n": 3}
    assert percentiles([]) is None
    assert percentiles(list(range(1, 101)), (50, 90, 99))["p99"] == 99


def test_the_device_gets_the_batch_s_common_stop_tokens_padded_to_a_fixed_length():
    from x0ne_engine_b200.engine.decode import STOP_IDS_ON_DEVICE, device_stop_ids
    row = lambda stops: Row(0, [1], SamplingParams(stop_token_ids=stops), 4, 0)   # noqa: E731
    pad = lambda ids: list(ids) + [-1] * (STOP_IDS_ON_DEVICE - len(ids))          # noqa: E731
    assert device_stop_ids([row((7, 3)), row((3, 7, 7))]) == pad([3, 7])
    assert device_stop_ids([row(()), row(())]) == pad([])
    assert device_stop_ids([row((7,)), row((8,))]) == pad([])                     # rows differ: the host decides alone
    assert device_stop_ids([row(tuple(range(STOP_IDS_ON_DEVICE + 1)))]) == pad([])
    assert len(device_stop_ids([row(tuple(range(STOP_IDS_ON_DEVICE)))])) == STOP_IDS_ON_DEVICE


def test_a_status_word_behind_the_picks_fails_the_step_it_came_with():
    """The decode loop reads, behind each step's picks, the word in which the tensor-core kernels
    report a wait that ran out.  With buffers filled by hand: steps whose word is zero give their
    picks; the step whose word is not zero raises, names itself, and clears the device's word."""
    import torch
    from x0ne_engine_b200.csrc.ops import KernelError
    from x0ne_engine_b200.engine.decode import DeviceBatch

    class Arrived:
        def synchronize(self):
            pass

    b = DeviceBatch.__new__(DeviceBatch)
    b._out_event = [Arrived(), Arrived()]
    b._out_host = [torch.tensor([11, 12, 13, 0, 99], dtype=torch.int32), torch.tensor([21, 22, 1 << 2, 0, 0], dtype=torch.int32)]
    b._batch_first = 6
    b.status = torch.tensor([1 << 2], dtype=torch.int32)
    assert b._read(6, 3) == [11, 12, 13]                     # the prompts' step of this batch: word 0
    with pytest.raises(KernelError, match=r"decode step 1 of this batch.*codes \[2\]"):
        b._read(7, 2)                                        # picks 21, 22 and a word that is not zero
    assert int(b.status[0]) == 0
    b._out_host[0][3] = 1 << 5
    with pytest.raises(KernelError, match=r"the prompts' step of this batch.*codes \[5\]"):
        b._read(6, 3)


def test_context_buckets_of_the_decode_graphs():
    """Decode graphs are kept per (rows, context bucket): powers of two from 2,048 up to the engine's limit."""
    from x0ne_engine_b200.engine.decode import DECODE_CONTEXT_BUCKET_MIN, context_bucket
    assert DECODE_CONTEXT_BUCKET_MIN == 2048
    assert context_bucket(1, 40960) == 2048 and context_bucket(2048, 40960) == 2048
    assert context_bucket(2049, 40960) == 4096 and context_bucket(8193, 40960) == 16384
    assert context_bucket(33000, 40960) == 40960           # the last bucket is the limit itself
    assert context_bucket(10, 512) == 512                  # an engine smaller than the smallest bucket
    seen = {context_bucket(n, 40960) for n in range(1, 40961, 7)}
    assert seen == {2048, 4096, 8192, 16384, 32768, 40960}
