"""The generation loop's decisions, with a fake engine: batching, stop tokens,
sequences that end earlier, slots given back and used again."""

import pytest

from flashdecode_cuda_b200.engine.generate import Backend, GenerationLoop, Request, plan_batch


class FakeEngine(Backend):
    """Produces token = (last fed token + 1) % 100 and logs every call."""

    def __init__(self, slots=4, tokens=256, block=16):
        self.slots, self.tokens, self.block = slots, tokens, block
        self.free = list(range(slots - 1, -1, -1))
        self.live = set()
        self.calls = []
        self.length = {}

    def capacity(self):
        return self.slots, self.tokens

    def tokens_held(self, n):
        return -(-n // self.block) * self.block

    def admit(self):
        s = self.free.pop()
        assert s not in self.live
        self.live.add(s)
        self.length[s] = 0
        return s

    def release(self, slot):
        assert slot in self.live, "released twice or never admitted"
        self.live.remove(slot)
        self.free.append(slot)

    def run(self, slots, tokens, requests, steps):
        assert len(set(slots)) == len(slots) and all(s in self.live for s in slots)
        self.calls.append((list(slots), [len(t) for t in tokens], list(steps)))
        for s, t in zip(slots, tokens):
            self.length[s] += len(t)
        return [(t[-1] + 1) % 100 for t in tokens]


def test_unequal_prompts_stop_tokens_and_length():
    eng = FakeEngine()
    reqs = [Request([1, 2, 3], 5, stop_token_ids=(6,), request_id=0),      # 4 5 6 -> stop at the 3rd
            Request([10], 2, request_id=1),                                # 11 12 -> length
            Request([50, 51], 4, stop_token_ids=(99,), request_id=2)]      # 52 53 54 55 -> length
    res = GenerationLoop(eng, max_batch=4).run(reqs)
    assert [r.tokens for r in res] == [[4, 5, 6], [11, 12], [52, 53, 54, 55]]
    assert [r.finish_reason for r in res] == ["stop", "length", "length"]
    # prompts in one step with unequal lengths, then one token each; the batch shrinks as requests end
    assert eng.calls[0][1] == [3, 1, 2]
    assert [len(c[0]) for c in eng.calls] == [3, 3, 2, 1]
    assert all(n == [1] * len(n) for _, n, _ in eng.calls[1:])
    assert eng.calls[2][2] == [2, 2]                                      # step counters of the live requests
    assert not eng.live and sorted(eng.free) == [0, 1, 2, 3]


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(slots=2)
    reqs = [Request([i], 1 + i % 3, request_id=i) for i in range(5)]
    res = GenerationLoop(eng, max_batch=8).run(reqs)
    assert [len(r.tokens) for r in res] == [1, 2, 3, 1, 2]
    firsts = [c for c in eng.calls if c[2] == [0] * len(c[2])]            # prompt steps
    assert [len(c[0]) for c in firsts] == [2, 2, 1]                        # no request joins a running batch
    used = {s for c in eng.calls for s in c[0]}
    assert used == {0, 1} and not eng.live


def test_batch_limited_by_cache_tokens():
    waiting = [Request([0] * 30, 10), Request([0] * 100, 20), Request([0] * 10, 5)]
    held = lambda n: -(-n // 16) * 16
    assert plan_batch(waiting, 8, 8, 48 + 128, held) == 2
    assert plan_batch(waiting, 8, 8, 48 + 127, held) == 1
    assert plan_batch(waiting, 1, 8, 10 ** 6, held) == 1
    assert plan_batch(waiting, 8, 2, 10 ** 6, held) == 2
    with pytest.raises(ValueError, match="cache holds"):
        plan_batch(waiting, 8, 8, 100, held)                              # the second can never fit


def test_slots_go_back_when_the_engine_fails():
    class Failing(FakeEngine):
        def run(self, *a):
            if len(self.calls) == 2:
                raise RuntimeError("boom")
            return super().run(*a)
    eng = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        GenerationLoop(eng).run([Request([1], 9, request_id=0), Request([2], 9, request_id=1)])
    assert not eng.live


def test_request_checks():
    with pytest.raises(ValueError):
        Request([], 3)
    with pytest.raises(ValueError):
        Request([1], 0)
    with pytest.raises(ValueError):
        GenerationLoop(FakeEngine(), max_batch=0)
