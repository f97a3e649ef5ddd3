"""The generation loop's decisions (no GPU), against a scripted stepper."""
import pytest

from cima_b200.engine import GenerationLoop, fit_prompt, plan_batches
from cima_b200.sampling import GenOptions


class Scripted:
    """Emits for each sequence its prompt's first token + 1, + 2, ...; records every call."""

    def __init__(self, max_batch=3, max_position=64, cache_tokens=64 * 4, page_size=64):
        self.max_batch, self.max_position, self.cache_tokens, self.page_size = max_batch, max_position, cache_tokens, page_size
        self.free = list(range(max_batch))
        self.calls = []
        self.base, self.count = {}, {}

    def open(self, n):
        assert n <= len(self.free)
        got, self.free = self.free[:n], self.free[n:]
        self.calls.append(("open", tuple(got)))
        return got

    def close(self, slots):
        assert not set(slots) & set(self.free)
        self.free = sorted(self.free + list(slots))
        self.calls.append(("close", tuple(slots)))

    def prefill(self, slots, prompts, options):
        self.calls.append(("prefill", tuple(slots), tuple(len(p) for p in prompts)))
        for s, p in zip(slots, prompts):
            self.base[s], self.count[s] = p[0], 0
        return self._next(slots)

    def decode(self, slots, last, options):
        self.calls.append(("decode", tuple(slots), tuple(last)))
        return self._next(slots)

    def _next(self, slots):
        out = []
        for s in slots:
            self.count[s] += 1
            out.append(self.base[s] + self.count[s])
        return out


def test_fit_prompt_keeps_first_token_and_tail():
    assert fit_prompt([1, 2, 3], 64) == ([1, 2, 3], False)
    p = list(range(100))
    got, cut = fit_prompt(p, 64)
    assert cut and len(got) == 48 and got[0] == 0 and got[1:] == p[-47:]
    with pytest.raises(ValueError):
        fit_prompt([], 64)


def test_plan_batches_respects_batch_size_and_cache():
    assert plan_batches([10, 10, 10, 10], 3, 64 * 8, 64) == [[0, 1, 2], [3]]
    assert plan_batches([65, 65, 64, 1], 8, 64 * 4, 64) == [[0, 1], [2, 3]]
    with pytest.raises(ValueError, match="may hold"):
        plan_batches([64 * 5], 8, 64 * 4, 64)


def test_budget_stop_and_early_finishers():
    st = Scripted()
    loop = GenerationLoop(st, eos_ids=[103])
    o = GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=5)
    res = loop.generate([[100, 7], [200], [300, 1, 2]], o)
    assert res[0].tokens == [101, 102] and res[0].finish_reason == "stop"        # 103 is a stop token, not emitted
    assert res[1].tokens == [201, 202, 203, 204, 205] and res[1].finish_reason == "length"
    assert res[2].tokens == [301, 302, 303, 304, 305]
    decodes = [c for c in st.calls if c[0] == "decode"]
    assert decodes[0][1] == (0, 1, 2) and decodes[2][1] == (1, 2)                # the stopped one left the batch
    assert decodes[0][2] == (101, 201, 301)
    assert len(decodes) == 4 and st.calls[-1] == ("close", (0, 1, 2))
    assert loop.stats.gen_tokens == 12 and loop.stats.batches == 1 and loop.stats.prompt_tokens == 6


def test_ignore_eos_and_per_request_options():
    st = Scripted()
    loop = GenerationLoop(st, eos_ids=[102])
    a = GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=3, ignore_eos=True)
    b = GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=4, stop=(203,))
    res = loop.generate([[100], [200]], [a, b])
    assert res[0].tokens == [101, 102, 103] and res[0].finish_reason == "length"
    assert res[1].tokens == [201, 202] and res[1].finish_reason == "stop"
    with pytest.raises(ValueError):
        loop.generate([[1]], [a, b])


def test_many_batches_one_after_another_and_slots_given_back_on_error():
    st = Scripted(max_batch=2)
    loop = GenerationLoop(st)
    res = loop.generate([[10 * i] for i in range(1, 6)], GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=2))
    assert [r.tokens for r in res] == [[10 * i + 1, 10 * i + 2] for i in range(1, 6)]
    assert [c for c in st.calls if c[0] == "open"] == [("open", (0, 1))] * 2 + [("open", (0,))]
    assert loop.stats.batches == 3 and st.free == [0, 1]

    class Failing(Scripted):
        def decode(self, slots, last, options):
            raise RuntimeError("boom")
    st = Failing()
    with pytest.raises(RuntimeError):
        GenerationLoop(st).generate([[1], [2]], GenOptions(max_tokens=3))
    assert st.free == [0, 1, 2]


def test_budget_is_capped_by_positions_and_zero_budget_needs_no_step():
    st = Scripted(max_position=20)
    loop = GenerationLoop(st)
    res = loop.generate([[5] * 4, [7] * 30], GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=100))
    assert len(res[0].tokens) == 16 and res[0].finish_reason == "length"          # 20 positions - 4 of the prompt
    # the long prompt was cut to first + tail so that 16 positions stay: 4 tokens, budget 16
    assert res[1].truncated and res[1].prompt_tokens == 4 and len(res[1].tokens) == 16
    res = loop.generate([[5]], GenOptions(max_tokens=0))
    assert res[0].tokens == [] and res[0].finish_reason == "length"
    assert not [c for c in st.calls[-1:] if c[0] == "prefill"]


def test_tokens_are_reported_as_their_steps_are_read():
    """``on_token`` gets every emitted token with its request's index, step by step in the order of the requests;
    a stop token is not reported; requests of a later batch follow those of the earlier one."""
    st = Scripted(max_batch=2)
    loop = GenerationLoop(st, eos_ids=[103])
    seen = []
    res = loop.generate([[100, 7], [200], [300]], GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=3),
                        on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 101), (1, 201), (0, 102), (1, 202), (1, 203), (2, 301), (2, 302), (2, 303)]
    assert [t for i, t in seen if i == 0] == res[0].tokens and res[0].finish_reason == "stop"
    loop.generate([[100]], GenOptions(temperature=0.0, repeat_penalty=1.0, max_tokens=2))        # no callback: none is kept
    assert len(seen) == 8
