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


class AheadBackend(FakeBackend):
    """The same arithmetic with steps that can be launched before the one before is read.  A token of None is
    taken from the step named in `after`, as the device would; the backend checks what a real one relies on:
    steps are collected in the order of their launches, at most two are in flight, a step launched ahead names
    the one launched just before it, and no slot is released while a step in flight still carries it."""
    runs_ahead = True

    def __init__(self, **kw):
        super().__init__(**kw)
        self.flying = []
        self.most_flying = 0
        self.rides = 0

    def launch_ahead(self, work, streams, params, after=None, rows_of=None):
        assert len(streams) == len(work) and len(self.flying) <= 1
        if after is not None:
            assert self.flying and self.flying[-1] is after and len(rows_of) == len(work)
        toks = []
        for k, (slot, tok) in enumerate(work):
            assert slot in self.sums, "stepped after its release"
            if tok is None:
                tok = after["picked"][rows_of[k]]
            toks.append(tok)
        self.steps.append([(s, [t]) for (s, _), t in zip(work, toks)])
        picked = []
        for (slot, _), tok in zip(work, toks):
            self.sums[slot] += tok
            picked.append(self.sums[slot] % 50)
        h = {"picked": picked, "slots": [s for s, _ in work]}
        self.flying.append(h)
        self.most_flying = max(self.most_flying, len(self.flying))
        return h

    def collect(self, h):
        assert self.flying and self.flying[0] is h, "collected out of order"
        self.flying.pop(0)
        return h["picked"], [float(p) for p in h["picked"]]

    def release(self, slot):
        assert all(slot not in h["slots"] for h in self.flying), "released while a step in flight carries it"
        super().release(slot)


@pytest.mark.parametrize("stop", [(), (40,), (6, 30), (10,)])
def test_one_step_ahead_gives_the_same_tokens(stop):
    prompts = [[10], [3], [1, 2, 3], [7, 7], [9]]
    budgets = [6, 2, 9, 1, 5]
    plain = generate(FakeBackend(max_seqs=3), prompts, budgets, stop_ids=stop)
    b = AheadBackend(max_seqs=3)
    seen = []
    ahead = generate(b, prompts, budgets, stop_ids=stop, on_token=lambda *a: seen.append(a))
    assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
    assert b.most_flying == 2 and not b.flying and not b.sums and sorted(b.free) == [0, 1, 2]
    # on_token sees every token once, in order, with the token that was fed in
    for i, r in enumerate(ahead):
        mine = [a for a in seen if a[0] == i]
        assert [a[1] for a in mine] == list(range(len(r.tokens))) and [a[3] for a in mine] == r.tokens
        assert [a[2] for a in mine] == [prompts[i][-1]] + r.tokens[:-1]
    # and with run_ahead off the backend's ordinary steps are used
    b2 = AheadBackend(max_seqs=3)
    off = generate(b2, prompts, budgets, stop_ids=stop, run_ahead=False)
    assert [r.tokens for r in off] == [r.tokens for r in plain] and b2.most_flying == 0


def test_a_stopped_request_rides_one_step_and_is_then_released():
    b = AheadBackend(max_seqs=2)
    res = generate(b, [[10], [3]], [6, 6], stop_ids=[40])       # request 0: 10, 20, 40 stop; request 1 runs on
    assert res[0].tokens == [10, 20, 40] and res[0].finish_reason == "stop"
    assert res[1].tokens == _expected([3], 6)
    # steps: prompts; then both; both; both (request 0 has stopped, unknown yet: it rides along); then request 1 alone
    assert [len(s) for s in b.steps] == [2, 2, 2, 2, 1, 1]
    assert not b.sums


def test_errors_while_running_ahead_give_every_slot_back():
    class Boom(AheadBackend):
        def collect(self, h):
            if len(self.steps) >= 4:
                self.flying.clear()
                raise RuntimeError("boom")
            return super().collect(h)

    b = Boom(max_seqs=3)
    with pytest.raises(RuntimeError):
        generate(b, [[1], [2], [3]], 8, stop_ids=[12])
    assert not b.sums and sorted(b.free) == [0, 1, 2]
