"""The generation loop's decisions, driven by a fake backend (no GPU)."""
import pytest

from stratum_b200.engine.generate import Backend, CapacityError, generate, plan_batches
from stratum_b200.sampling import Pcg32, SamplingParams


class FakeBackend(Backend):
    """Next token = (sum of all tokens the sequence has been fed) % 50; records every step."""

    def __init__(self, n_pages=8, max_seqs=4):
        self.n_pages, self.max_seqs = n_pages, max_seqs
        self.free = list(range(max_seqs))
        self.sums = {}
        self.steps = []
        self.held_max = 0

    def acquire(self):
        s = min(self.free)
        self.free.remove(s)
        self.sums[s] = 0
        self.held_max = max(self.held_max, len(self.sums))
        return s

    def release(self, slot):
        assert slot in self.sums, "released twice"
        del self.sums[slot]
        self.free.append(slot)

    def step_and_pick(self, work, streams, params):
        assert len(streams) == len(work)
        self.steps.append([(s, list(t)) for s, t in work])
        out = []
        for s, toks in work:
            self.sums[s] += sum(toks)
            out.append(self.sums[s] % 50)
        return out, [float(o) for o in out]


def _expected(prompt, n, stop=()):
    seq, total, out = list(prompt), sum(prompt), []
    for _ in range(n):
        t = total % 50
        out.append(t)
        if t in stop:
            break
        total += t
    return out


def test_prompts_in_one_step_then_one_token_each():
    b = FakeBackend()
    prompts = [[1, 2, 3], [7], [5, 5, 5, 5]]
    res = generate(b, prompts, 4)
    assert [r.tokens for r in res] == [_expected(p, 4) for p in prompts]
    assert all(r.finish_reason == "length" for r in res)
    assert [len(t) for _, t in b.steps[0]] == [3, 1, 4]              # unequal prompts, one step
    assert all(len(t) == 1 for step in b.steps[1:] for _, t in step)
    assert len(b.steps) == 4                                       # the 4th token is picked, never fed back
    assert not b.sums and sorted(b.free) == [0, 1, 2, 3]             # every slot given back once


def test_stop_tokens_and_early_leavers():
    b = FakeBackend()
    prompts = [[10], [3]]                 # 10 -> 10, 20, 40, 30(80%50) ...;  3 -> 3, 6, 12, 24, 48
    res = generate(b, prompts, [6, 2], stop_ids=[40])
    assert res[0].tokens == [10, 20, 40] and res[0].finish_reason == "stop"
    assert res[1].tokens == [3, 6] and res[1].finish_reason == "length"
    # request 1 left after two tokens: the third step runs request 0 alone
    assert [len(s) for s in b.steps] == [2, 2, 1]
    assert not b.sums


def test_batches_follow_one_another_and_reuse_slots():
    b = FakeBackend(n_pages=8, max_seqs=2)
    prompts = [[i + 1] for i in range(5)]
    res = generate(b, prompts, 3)
    assert [r.tokens for r in res] == [_expected(p, 3) for p in prompts]
    assert b.held_max == 2
    assert [len(s) for s in b.steps] == [2, 2, 2, 2, 2, 2, 1, 1, 1]   # 2 + 2 + 1 requests, 3 steps a batch
    assert {slot for step in b.steps for slot, _ in step} == {0, 1}   # the same slots serve every batch


def test_plan_respects_pages_and_refuses_the_impossible():
    assert plan_batches([64, 64, 64], [1, 1, 1], n_pages=2, max_seqs=8) == [[0, 1], [2]]
    assert plan_batches([64, 64], [2, 2], n_pages=4, max_seqs=8) == [[0, 1]]          # 65 keys -> 2 pages each
    assert plan_batches([1] * 5, [1] * 5, n_pages=100, max_seqs=8, max_batch=2) == [[0, 1], [2, 3], [4]]
    with pytest.raises(CapacityError, match="exceeds KV capacity"):
        plan_batches([200], [100], n_pages=4, max_seqs=8)
    with pytest.raises(ValueError, match="empty prompt"):
        plan_batches([0], [1], n_pages=4, max_seqs=8)


def test_zero_budget_and_slots_released_on_error():
    b = FakeBackend()
    res = generate(b, [[1], [2]], [0, 2])
    assert res[0].tokens == [] and res[0].finish_reason == "length" and res[1].tokens == _expected([2], 2)

    class Boom(FakeBackend):
        def step_and_pick(self, work, streams, params):
            if len(self.steps) == 1:
                raise RuntimeError("boom")
            return super().step_and_pick(work, streams, params)

    b = Boom()
    with pytest.raises(RuntimeError):
        generate(b, [[1], [2]], 5)
    assert not b.sums and sorted(b.free) == [0, 1, 2, 3]


def test_streams_belong_to_requests_not_to_batches():
    seen = {}

    class Rec(FakeBackend):
        def step_and_pick(self, work, streams, params):
            for (slot, toks), st in zip(work, streams):
                seen.setdefault(id(st), []).append(st.uniform())
            return super().step_and_pick(work, streams, params)

    p = SamplingParams(temperature=0.8, seed=11)
    generate(Rec(max_seqs=4), [[1], [2], [3]], 3, params=p)
    together = sorted(seen.values())
    seen.clear()
    generate(Rec(max_seqs=1), [[1], [2], [3]], 3, params=p)
    assert sorted(seen.values()) == together
    assert together[0][:2] != together[1][:2]
    assert Pcg32(11, 2).uniform() in [v[0] for v in together]
