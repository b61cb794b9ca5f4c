"""The generation loop's decisions, against a scripted backend (no GPU)."""
import pytest

from mynah_slm_b200.engine.generate import (GenerationError, Request, Timing, generate, plan_batches, tokens_held)


class Scripted:
    """Each sequence emits prompt[0]+1, +2, ...; records what the loop asks of it."""

    def __init__(self, budget=64 * 64, max_positions=4096, n_slots=8):
        self.max_positions = max_positions
        self.budget = budget
        self.free_slots = list(range(n_slots - 1, -1, -1))
        self.state = {}
        self.log = []
        self.opened = []

    def free_tokens(self):
        return self.budget

    def open(self, request_index, prompt):
        slot = self.free_slots.pop()
        self.state[slot] = [prompt[0], len(prompt)]
        self.opened.append((request_index, slot))
        return slot

    def close(self, slot):
        assert slot in self.state, "closed twice"
        del self.state[slot]
        self.free_slots.append(slot)
        self.log.append(("close", slot))

    def _next(self, slot):
        self.state[slot][0] += 1
        return self.state[slot][0]

    def prefill(self, slots, prompts):
        self.log.append(("prefill", tuple(slots), tuple(len(p) for p in prompts)))
        return [self._next(s) for s in slots]

    def decode(self, slots, tokens):
        for s, t in zip(slots, tokens):
            assert t == self.state[s][0], "the loop must feed back the token it was given"
            self.state[s][1] += 1
        self.log.append(("decode", tuple(slots)))
        return [self._next(s) for s in slots]


def test_unequal_prompts_and_early_end():
    be = Scripted()
    reqs = [Request([100, 1, 2], 5), Request([200], 2), Request([300] * 7, 4)]
    out = generate(be, reqs, max_batch=8)
    assert [r.tokens for r in out] == [[101, 102, 103, 104, 105], [201, 202], [301, 302, 303, 304]]
    assert [r.finish_reason for r in out] == ["length"] * 3
    steps = [e for e in be.log if e[0] in ("prefill", "decode")]
    assert steps[0] == ("prefill", (0, 1, 2), (3, 1, 7))          # all prompts in ONE step
    assert steps[1] == ("decode", (0, 1, 2))
    assert steps[2] == ("decode", (0, 2))                          # the 2-token request has left
    assert steps[-1] == ("decode", (0,))
    assert not be.state                                            # every slot given back


def test_stop_token_is_counted_not_emitted():
    be = Scripted()
    out = generate(be, [Request([10], 10), Request([20], 10)], stop_ids=[13, 22])
    assert out[0].tokens == [11, 12] and out[0].produced == 3 and out[0].finish_reason == "stop"
    assert out[1].tokens == [21] and out[1].produced == 2 and out[1].finish_reason == "stop"


def test_first_token_can_stop():
    be = Scripted()
    out = generate(be, [Request([10], 10)], stop_ids=[11])
    assert out[0].tokens == [] and out[0].produced == 1 and out[0].finish_reason == "stop"
    assert [e[0] for e in be.log] == ["prefill", "close"]


def test_batches_follow_one_another_and_reuse_slots():
    be = Scripted(n_slots=2)
    reqs = [Request([100 * (i + 1)], 1 + i) for i in range(5)]
    out = generate(be, reqs, max_batch=2)
    assert [r.tokens for r in out] == [[100 * (i + 1) + k + 1 for k in range(1 + i)] for i in range(5)]
    prefills = [e for e in be.log if e[0] == "prefill"]
    assert len(prefills) == 3                                       # 2 + 2 + 1 requests
    assert {s for _, s in be.opened} == {0, 1}                      # five requests, two slots
    # no request of the second batch starts before the first batch is over
    first_close_all = max(i for i, e in enumerate(be.log) if e == ("close", 1) or e == ("close", 0))
    assert be.log.index(prefills[1]) > be.log.index(prefills[0])


def test_cache_budget_limits_a_batch():
    reqs = [Request([1] * 60, 10), Request([1] * 60, 10), Request([1] * 10, 3)]
    assert tokens_held(60, 10, 4096) == 128
    assert plan_batches(reqs, max_batch=8, budget_tokens=256, max_positions=4096) == [[0, 1], [2]]
    assert plan_batches(reqs, max_batch=8, budget_tokens=1024, max_positions=4096) == [[0, 1, 2]]
    with pytest.raises(GenerationError, match="may hold 128 tokens"):
        plan_batches(reqs, max_batch=8, budget_tokens=64, max_positions=4096)
    with pytest.raises(GenerationError, match="empty prompt"):
        plan_batches([Request([], 3)], 8, 1024, 4096)
    with pytest.raises(GenerationError, match="exceeds the model"):
        plan_batches([Request([1] * 50, 3)], 8, 1024, max_positions=40)


def test_zero_new_tokens_and_context_end():
    be = Scripted(max_positions=6)
    out = generate(be, [Request([1, 2, 3], 0), Request([50, 1, 1, 1], 10)])
    assert out[0].tokens == [] and out[0].finish_reason == "length"
    # prompt of 4 in a context of 6: positions 4 and 5 take two more inputs
    assert out[1].tokens == [51, 52, 53] and out[1].finish_reason == "context"
    assert all(e[1] != (0,) or e[0] != "prefill" or True for e in be.log)


def test_callback_stops_one_sequence():
    be = Scripted()
    seen = []

    def cb(i, tok):
        seen.append((i, tok))
        return 1 if (i, tok) == (0, 12) else 0

    out = generate(be, [Request([10], 5), Request([20], 3)], callback=cb)
    assert out[0].tokens == [11, 12] and out[0].finish_reason == "callback"
    assert out[1].tokens == [21, 22, 23]
    assert (1, 23) in seen


def test_timing_line():
    be = Scripted()
    t = Timing(load_s=0.5, device_name="B200")
    generate(be, [Request([1, 2, 3], 4), Request([9], 2)], timing=t)
    assert t.n_prompt == 4 and t.n_gen == 6 and t.ttft_s > 0
    line = t.format()
    assert line.startswith("[load 0.50s | prompt 4 tok, prefill ") and "gen 6 tok, decode " in line and "TTFT" in line


def test_slots_are_given_back_when_a_step_fails():
    class Failing(Scripted):
        def decode(self, slots, tokens):
            raise RuntimeError("boom")
    be = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate(be, [Request([1], 5), Request([2], 5)])
    assert not be.state


# ---------------------------------------------------------------- one step ahead

class ScriptedAhead(Scripted):
    """The same scripted sequences behind the launch/collect pair: a launched step's result stays "on the
    device" (in the handle) until it is collected, and a later launch may be fed from it row by row."""
    runs_ahead = True

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.in_flight = 0

    def decode(self, slots, tokens):
        raise AssertionError("a backend that runs ahead is not driven step by step")

    def decode_launch(self, slots, tokens=None, feed=None):
        if feed is not None:
            prev, rows = feed
            assert tokens is None and len(rows) == len(slots)
            tokens = [prev["tokens"][j] for j in rows]          # taken "on the device"
        for s, t in zip(slots, tokens):
            assert s in self.state, "a closed slot is stepped"
            assert t == self.state[s][0], "the step must be fed the token sampled for this sequence"
            assert self.state[s][1] < self.max_positions, "a step beyond the last position"
            self.state[s][1] += 1
        self.in_flight += 1
        assert self.in_flight <= 2
        self.log.append(("decode", tuple(slots)))
        return {"tokens": [self._next(s) for s in slots], "collected": False}

    def decode_collect(self, h):
        assert not h["collected"]
        h["collected"] = True
        self.in_flight -= 1
        return list(h["tokens"])


SCENARIOS = [
    dict(reqs=[([100, 1, 2], 5), ([200], 2), ([300] * 7, 4)], kw={}),
    dict(reqs=[([10], 10), ([20], 10)], kw=dict(stop_ids=[13, 22])),
    dict(reqs=[([10], 10)], kw=dict(stop_ids=[11])),
    dict(reqs=[([100 * (i + 1)], 1 + i) for i in range(5)], kw=dict(max_batch=2), n_slots=2),
    dict(reqs=[([1, 2, 3], 0), ([50, 1, 1, 1], 10)], kw={}, max_positions=6),
    dict(reqs=[([10], 5), ([20], 3), ([30], 1), ([40], 9)], kw=dict(stop_ids=[43, 12])),
]


@pytest.mark.parametrize("sc", SCENARIOS)
def test_one_step_ahead_gives_the_step_by_step_results(sc):
    outs = []
    for cls in (Scripted, ScriptedAhead):
        be = cls(max_positions=sc.get("max_positions", 4096), n_slots=sc.get("n_slots", 8))
        seen = []
        out = generate(be, [Request(list(p), n) for p, n in sc["reqs"]], callback=lambda i, t: seen.append((i, t)) or 0, **sc["kw"])
        assert not be.state                                                       # every slot given back, once
        outs.append(([(r.tokens, r.produced, r.finish_reason) for r in out], sorted(seen), be))
    assert outs[0][0] == outs[1][0] and outs[0][1] == outs[1][1]
    assert outs[1][2].in_flight == 0


def test_one_step_ahead_runs_a_stopped_sequence_one_row_more_and_no_certain_end():
    be = ScriptedAhead()
    out = generate(be, [Request([10], 10), Request([20], 3)], stop_ids=[12])
    assert out[0].tokens == [11] and out[0].finish_reason == "stop" and out[1].tokens == [21, 22, 23]
    steps = [e for e in be.log if e[0] in ("decode", "close")]
    # step 1 samples 12 (stop) for slot 0, but step 2 was already launched with it; it is closed after that step.
    # Slot 1 samples its third and last token in step 2, which is known beforehand: there is no step 3.
    assert steps == [("decode", (0, 1)), ("decode", (0, 1)), ("close", 0), ("close", 1)]


def test_one_step_ahead_callback_and_failure():
    be = ScriptedAhead()
    out = generate(be, [Request([10], 5), Request([20], 3)], callback=lambda i, t: 1 if (i, t) == (0, 12) else 0)
    assert out[0].tokens == [11, 12] and out[0].finish_reason == "callback" and out[1].tokens == [21, 22, 23]
    assert not be.state

    class Failing(ScriptedAhead):
        def decode_collect(self, h):
            raise RuntimeError("boom")
    be = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate(be, [Request([1], 5), Request([2], 5)])
    assert not be.state
