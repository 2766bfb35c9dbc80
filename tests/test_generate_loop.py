"""The generation loop's decisions, against a scripted engine (no GPU)."""
import pytest
import torch

from qwen_triton_b200.engine.generate import finish_reason, generate, plan_batches
from qwen_triton_b200.engine.step import plan_passes
from qwen_triton_b200.sampling import SamplingParams, uniform_for


class ScriptedEngine:
    """Next token = (last token + 1) % vocab.  Records every step and checks slot discipline."""

    device = "cpu"

    def __init__(self, vocab=50, num_slots=3, total_pages=6, page_tokens=4, max_seq_len=24, eos=(49,)):
        self.vocab, self.num_slots, self.total_pages, self.page_tokens = vocab, num_slots, total_pages, page_tokens
        self.max_seq_len, self.eos_token_ids = max_seq_len, eos
        self.free = list(range(num_slots))
        self.lengths: dict[int, int] = {}
        self.steps: list[list[tuple[int, int]]] = []
        self.slot_history: list[int] = []

    def new_sequence(self):
        slot = self.free.pop(0)
        self.lengths[slot] = 0
        self.slot_history.append(slot)
        return slot

    def release(self, slot):
        assert slot in self.lengths, "released twice"
        del self.lengths[slot]
        self.free.append(slot)

    def check_kernels(self, wait=True):
        pass

    def step(self, entries):
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        logits = torch.zeros(len(entries), self.vocab)
        for row, entry in enumerate(entries):
            assert entry.want == [len(entry.tokens) - 1]
            self.lengths[entry.slot] += len(entry.tokens)
            assert self.lengths[entry.slot] <= self.max_seq_len
            pages = sum(-(-n // self.page_tokens) for n in self.lengths.values())
            assert pages <= self.total_pages
            logits[row, (entry.tokens[-1] + 1) % self.vocab] = 1.0
        return logits


class ArgmaxSampler:
    def __init__(self):
        self.calls = []

    def sample(self, logits, params, requests, steps):
        self.calls.append((list(requests), list(steps)))
        return logits.argmax(dim=-1).tolist()


def test_unequal_prompts_stop_tokens_and_early_finish():
    engine, sampler = ScriptedEngine(), ArgmaxSampler()
    prompts = [[10, 11, 12], [46], [20, 21]]
    results = generate(engine, prompts, max_new_tokens=5, sampler=sampler)
    assert results[0].tokens == [13, 14, 15, 16, 17] and results[0].finish_reason == "length"
    assert results[1].tokens == [47, 48, 49] and results[1].finish_reason == "stop"       # the stop token is emitted
    assert results[2].tokens == [22, 23, 24, 25, 26]
    # one prefill step with the three prompts, then one token each; the stopped sequence leaves the batch
    assert engine.steps[0] == [(0, 3), (1, 1), (2, 2)]
    assert engine.steps[1] == [(0, 1), (1, 1), (2, 1)] and engine.steps[3] == [(0, 1), (2, 1)]
    assert len(engine.steps) == 5 and not engine.lengths and sorted(engine.free) == [0, 1, 2]
    assert sampler.calls[0] == ([0, 1, 2], [0, 0, 0]) and sampler.calls[3] == ([0, 2], [3, 3])


class PlanningEngine(ScriptedEngine):
    """The scripted engine with the two halves of a one-token step: ``plan_decode`` gives every planned sequence
    its next position, ``run_planned`` takes the tokens.  It checks that a position is given exactly once."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.plans: list[tuple[list[int], bool]] = []
        self.fed: dict[int, int] = {}            # tokens fed per slot, which must equal its length after every step

    def new_sequence(self):
        slot = super().new_sequence()
        self.fed[slot] = 0
        return slot

    def step(self, entries):
        for entry in entries:
            self.fed[entry.slot] += len(entry.tokens)
        return super().step(entries)

    def plan_decode(self, slots, extend=True):
        self.plans.append((list(slots), extend))
        for slot in slots:
            assert slot in self.lengths, "planned for a slot that is not in use"
            if extend:
                self.lengths[slot] += 1
            assert self.lengths[slot] == self.fed[slot] + 1, "a planned sequence has exactly one position it has not been fed"
            assert self.lengths[slot] <= self.max_seq_len
        return list(slots)

    def run_planned(self, plan, tokens):
        assert len(plan) == len(tokens)
        self.steps.append([(slot, 1) for slot in plan])
        logits = torch.zeros(len(plan), self.vocab)
        for row, (slot, token) in enumerate(zip(plan, tokens)):
            self.fed[slot] += 1
            assert self.fed[slot] == self.lengths[slot]
            logits[row, (token + 1) % self.vocab] = 1.0
        return logits


class LaunchSampler(ArgmaxSampler):
    def launch(self, logits, params, requests, steps):
        tokens = self.sample(logits, params, requests, steps)

        class Pending:
            def tokens(self):
                return tokens

        return Pending()


class PipelinedEngine(PlanningEngine):
    """Takes the chosen tokens as a tensor and row numbers, as the engine does when the next step is queued before
    the host has read them."""

    accepts_chosen_tokens = True

    def run_planned(self, plan, tokens, chosen=None):
        if chosen is not None:
            tokens = [int(chosen[row]) for row in tokens]
        return super().run_planned(plan, tokens)


class DeviceSampler(LaunchSampler):
    def launch(self, logits, params, requests, steps):
        pending = super().launch(logits, params, requests, steps)
        pending.device = torch.tensor(pending.tokens(), dtype=torch.int32)
        return pending


def test_steps_queued_ahead_give_the_same_tokens_and_drop_the_rows_of_stopped_requests():
    plain_engine, engine = ScriptedEngine(), PipelinedEngine()
    prompts = [[10, 11, 12], [46], [20, 21]]
    expected = generate(plain_engine, prompts, max_new_tokens=5, sampler=ArgmaxSampler())
    sampler = DeviceSampler()
    results = generate(engine, prompts, max_new_tokens=5, sampler=sampler)
    assert [(r.tokens, r.finish_reason) for r in results] == [(r.tokens, r.finish_reason) for r in expected]
    # every plan is run at once (no plan is made twice); slot 1 stops at its third token, when the step for its fourth
    # is already queued: it runs with three rows and the row of slot 1 is dropped
    assert engine.plans == [([0, 1, 2], True)] * 3 + [([0, 2], True)]
    assert engine.steps == [[(0, 3), (1, 1), (2, 2)], [(0, 1), (1, 1), (2, 1)], [(0, 1), (1, 1), (2, 1)], [(0, 1), (1, 1), (2, 1)],
                            [(0, 1), (2, 1)]]
    assert sampler.calls[3] == ([0, 1, 2], [3, 3, 3]) and sampler.calls[4] == ([0, 2], [4, 4])
    assert not engine.lengths and sorted(engine.free) == [0, 1, 2]
    # the same through several batches, the cache's end, and with the pipeline switched off by the environment
    engine = PipelinedEngine(num_slots=2, total_pages=100)
    results = generate(engine, [[1], [2, 3], [4], [5, 6, 7], [8]], max_new_tokens=2, sampler=DeviceSampler(), ignore_eos=True)
    assert [r.tokens for r in results] == [[2, 3], [4, 5], [5, 6], [8, 9], [9, 10]] and engine.slot_history == [0, 1, 0, 1, 0]
    engine = PipelinedEngine(max_seq_len=6, total_pages=10)
    result = generate(engine, [[1, 2, 3, 4]], max_new_tokens=10, sampler=DeviceSampler(), ignore_eos=True)[0]
    assert result.tokens == [5, 6, 7] and result.finish_reason == "max_seq_len"


def test_the_pipeline_can_be_switched_off(monkeypatch):
    monkeypatch.setenv("QT_B200_PIPELINE", "0")
    engine = PipelinedEngine()
    results = generate(engine, [[10, 11, 12], [46], [20, 21]], max_new_tokens=5, sampler=DeviceSampler())
    assert [r.tokens for r in results] == [[13, 14, 15, 16, 17], [47, 48, 49], [22, 23, 24, 25, 26]]
    assert engine.plans[3] == ([0, 2], False)              # planned again after the stop token, as without a pipeline


def test_the_next_step_is_planned_ahead_and_replanned_after_a_stop_token():
    plain_engine, engine = ScriptedEngine(), PlanningEngine()
    prompts = [[10, 11, 12], [46], [20, 21]]
    expected = generate(plain_engine, prompts, max_new_tokens=5, sampler=ArgmaxSampler())
    results = generate(engine, prompts, max_new_tokens=5, sampler=LaunchSampler())
    assert [(r.tokens, r.finish_reason) for r in results] == [(r.tokens, r.finish_reason) for r in expected]
    assert engine.steps == plain_engine.steps            # the same sequences run at every step
    # planned after the prompts and after every step while someone can go on; when slot 1 stops at its third token
    # the plan for three is dropped and made again, without a second position, for the two that go on
    assert engine.plans[:2] == [([0, 1, 2], True), ([0, 1, 2], True)]
    assert ([0, 1, 2], True) == engine.plans[2] and engine.plans[3] == ([0, 2], False)
    assert engine.plans[4] == ([0, 2], True) and len(engine.plans) == 5      # the last tokens end by count: nothing to plan
    assert not engine.lengths and sorted(engine.free) == [0, 1, 2]


def test_planning_stops_at_the_cache_end_and_survives_batches():
    engine = PlanningEngine(max_seq_len=6, total_pages=10)
    result = generate(engine, [[1, 2, 3, 4]], max_new_tokens=10, sampler=LaunchSampler(), ignore_eos=True)[0]
    assert result.tokens == [5, 6, 7] and result.finish_reason == "max_seq_len"
    assert engine.plans == [([0], True), ([0], True)]     # the third new token cannot be fed back: no plan for it
    engine = PlanningEngine(num_slots=2, total_pages=100)
    results = generate(engine, [[1], [2, 3], [4], [5, 6, 7], [8]], max_new_tokens=2, sampler=LaunchSampler(), ignore_eos=True)
    assert [r.tokens for r in results] == [[2, 3], [4, 5], [5, 6], [8, 9], [9, 10]]
    assert engine.slot_history == [0, 1, 0, 1, 0]


def test_more_requests_than_slots_run_as_batches_and_reuse_slots():
    engine = ScriptedEngine(num_slots=2, total_pages=100)
    prompts = [[1], [2, 3], [4], [5, 6, 7], [8]]
    results = generate(engine, prompts, max_new_tokens=2, sampler=ArgmaxSampler(), ignore_eos=True)
    assert [r.tokens for r in results] == [[2, 3], [4, 5], [5, 6], [8, 9], [9, 10]]
    assert engine.slot_history == [0, 1, 0, 1, 0]
    assert [len(s) for s in engine.steps] == [2, 2, 2, 2, 1, 1]


def test_batches_respect_the_cache_size():
    batches = plan_batches([5, 9, 17, 3], 8, page_tokens=4, total_pages=12, num_slots=8, max_seq_len=64)
    # pages at final length: 4, 5, 7, 3
    assert batches == [[0, 1], [2, 3]]
    assert plan_batches([5, 9, 17, 3], 8, page_tokens=4, total_pages=100, num_slots=8, max_seq_len=64,
                        max_batch_size=3) == [[0, 1, 2], [3]]
    with pytest.raises(ValueError, match="cache pages"):
        plan_batches([100], 8, page_tokens=4, total_pages=12, num_slots=8, max_seq_len=200)
    with pytest.raises(ValueError, match="max_seq_len"):
        plan_batches([100], 8, page_tokens=4, total_pages=120, num_slots=8, max_seq_len=64)
    with pytest.raises(ValueError, match="empty"):
        plan_batches([0], 8, page_tokens=4, total_pages=12, num_slots=8, max_seq_len=64)
    engine = ScriptedEngine(num_slots=3, total_pages=6, page_tokens=4, max_seq_len=24)
    generate(engine, [[1] * 5, [2] * 6, [3] * 2], max_new_tokens=3, sampler=ArgmaxSampler(), ignore_eos=True)
    assert engine.steps[0] == [(0, 5), (1, 6)]           # 2 + 3 pages fit, the third request waits for the next batch


def test_sequence_ends_where_the_cache_ends():
    engine = ScriptedEngine(max_seq_len=6, total_pages=10)
    result = generate(engine, [[1, 2, 3, 4]], max_new_tokens=10, sampler=ArgmaxSampler(), ignore_eos=True)[0]
    # positions 0..5 can be held: the prompt and two fed-back tokens; the third new token cannot be fed back
    assert result.tokens == [5, 6, 7] and result.finish_reason == "max_seq_len"
    assert finish_reason(3, 1, 5, stop_ids=frozenset({3}), max_new_tokens=4, max_seq_len=10) == "stop"
    assert finish_reason(2, 4, 5, stop_ids=frozenset({3}), max_new_tokens=4, max_seq_len=10) == "length"
    assert finish_reason(2, 1, 5, stop_ids=frozenset({3}), max_new_tokens=4, max_seq_len=10) == ""


def test_stop_ids_and_eos_switch():
    engine = ScriptedEngine(eos=(12,))
    assert generate(engine, [[10]], max_new_tokens=5, sampler=ArgmaxSampler())[0].tokens == [11, 12]
    assert generate(engine, [[10]], max_new_tokens=5, sampler=ArgmaxSampler(), ignore_eos=True)[0].tokens == [11, 12, 13, 14, 15]
    out = generate(engine, [[10]], max_new_tokens=5, sampler=ArgmaxSampler(), ignore_eos=True, stop_token_ids=[14])[0]
    assert out.tokens == [11, 12, 13, 14] and out.finish_reason == "stop"
    assert generate(engine, [[10]], max_new_tokens=0, sampler=ArgmaxSampler())[0].tokens == []


def test_slots_go_back_when_a_step_fails():
    engine = ScriptedEngine()

    def broken(entries):
        raise RuntimeError("boom")

    engine.step = broken
    with pytest.raises(RuntimeError, match="boom"):
        generate(engine, [[1], [2]], max_new_tokens=2, sampler=ArgmaxSampler())
    assert not engine.lengths and sorted(engine.free) == [0, 1, 2]


def test_passes_cut_by_total_and_by_chunk():
    def sizes(passes):
        return [[(p.entry, p.begin, p.end) for p in pieces] for pieces in passes]

    assert sizes(plan_passes([5, 9, 17], 100, None)) == [[(0, 0, 5), (1, 0, 9), (2, 0, 17)]]
    assert sizes(plan_passes([5, 9, 17], 10, None)) == [[(0, 0, 5), (1, 0, 5)], [(1, 5, 9), (2, 0, 6)], [(2, 6, 16)], [(2, 16, 17)]]
    assert sizes(plan_passes([5, 9], 100, 4)) == [[(0, 0, 4), (1, 0, 4)], [(0, 4, 5), (1, 4, 8)], [(1, 8, 9)]]
    assert sizes(plan_passes([1, 1, 1], 2, None)) == [[(0, 0, 1), (1, 0, 1)], [(2, 0, 1)]]


def test_uniform_stream_matches_the_plain_reference():
    import plain_qwen3 as plain
    for seed, request, step in ((0, 0, 0), (1, 3, 9), (2 ** 40 + 5, 17, 255)):
        assert uniform_for(seed, request, step) == plain.uniform_for(seed, request, step)
    assert SamplingParams().temperature == 0.0
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)


def test_sampling_parameters_are_checked():
    import pytest
    from qwen_triton_b200.sampling import SamplingParams
    assert SamplingParams().top_k == 0 and SamplingParams().top_p == 1.0
    for bad in (dict(temperature=-0.1), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
