"""The engine's step logic without a GPU: the real scheduler and cache manager
under ``Engine.step``, with a stand-in for the model runner whose "model"
answers every fed token with a number that depends only on the request and
the token's position.  What is checked is the bookkeeping around steps that
are launched ahead: which launched steps are taken, which are dropped, and
that the outputs are the same as without launching ahead."""
from types import SimpleNamespace

import numpy as np
import pytest

from railgun_b200.cache.manager import PageAllocator
from railgun_b200.engine.engine import Engine
from railgun_b200.engine.request import SamplingParams
from railgun_b200.engine.scheduler import Scheduler, SchedulerConfig, SchedulerError


def answer(rid: int, position: int) -> int:
    """The token the stand-in model gives after the token at ``position`` of request ``rid``."""
    return (rid * 31 + position * 7 + (position * position) % 11) % 97


class StandInRunner:
    """What ``Engine`` uses of a ModelRunner.  Like the real one, a decode step launched through
    ``decode_step_flat`` advances its requests at once, a step launched ahead commits nothing."""
    use_graphs = True

    def __init__(self, alloc):
        self.alloc = alloc
        self.last_greedy = None
        self.log = []

    def decode_step_flat(self, ids, tokens):
        pos = [self.alloc.num_computed(int(r)) for r in ids]
        for r, p in zip(ids, pos):
            self.alloc.reserve(int(r), p + 1)
        self.alloc.advance(np.ascontiguousarray(ids, dtype=np.int64), 1)
        self._host = np.array([answer(int(r), p) for r, p in zip(ids, pos)], dtype=np.int32)
        self.last_greedy = True
        self.log.append(("step", tuple(int(r) for r in ids)))

    def greedy_tokens_host(self):
        return self._host

    def check_device_errors(self):
        pass

    def decode_follow(self, ids, after):
        ahead = 0 if after is None else 1
        pos = [self.alloc.num_computed(int(r)) + ahead for r in ids]
        for r, p in zip(ids, pos):
            if not self.alloc.can_reserve(int(r), p + 1):
                return None
        for r, p in zip(ids, pos):
            self.alloc.reserve(int(r), p + 1)
        toks = np.array([answer(int(r), p) for r, p in zip(ids, pos)], dtype=np.int32)
        self.log.append(("ahead", tuple(int(r) for r in ids)))
        return SimpleNamespace(ids=np.array(ids, dtype=np.int64), tokens=lambda: toks)

    def step(self, batch):
        self.last_greedy = None
        out = []
        for e in batch:
            start = self.alloc.num_computed(e.request_id) if self.alloc.has(e.request_id) else 0
            if not self.alloc.has(e.request_id):
                self.alloc.add_request(e.request_id)
            self.alloc.reserve(e.request_id, start + len(e.tokens))
            out += [answer(e.request_id, start + w) for w in e.want]
        self.log.append(("mixed", tuple(e.request_id for e in batch)))
        return np.array(out, dtype=np.int32) if out else None


def make_engine(run_ahead, pages=64, page=4, seats=3, budget=32):
    eng = Engine.__new__(Engine)
    alloc = PageAllocator([page], [pages], [0], seats)
    eng.runner = StandInRunner(alloc)
    eng.scheduler = Scheduler(alloc, SchedulerConfig(budget, seats, 0, 512))
    eng.sampler = SimpleNamespace(sample_arrays=lambda logits, sp: logits)             # the stand-in's logits are tokens
    eng._next_id, eng.steps_run = 1, 0
    eng.run_ahead, eng._ahead, eng.steps_ahead = run_ahead, None, 0
    eng.runner.model = SimpleNamespace(vocab_size=97)
    return eng


def expected_output(rid, prompt, n, stop=()):
    toks, out = list(prompt), []
    for _ in range(n):
        t = answer(rid, len(toks) - 1)
        out.append(t)
        toks.append(t)
        if t in stop:
            break
    return out


def drive(eng, script):
    """``script``: step number -> callable(engine) run before that step (arrivals, aborts)."""
    trace, k = [], 0
    while eng.has_unfinished() or k in script or any(s > k for s in script):
        if k in script:
            script[k](eng)
        out = eng.step()
        trace.append(sorted(out) if out else out)
        k += 1
        assert k < 500
    return trace


@pytest.mark.parametrize("pages", [64, 14])
def test_steps_launched_ahead_change_nothing_in_the_bookkeeping(pages):
    prompts = {1: [3, 4, 5], 2: [9] * 7, 3: [1], 4: [8, 8, 8, 8, 8], 5: [2, 6]}
    stop2 = expected_output(2, prompts[2], 20)[6]                # request 2 ends on a stop token
    params = {1: SamplingParams(max_new_tokens=25), 2: SamplingParams(max_new_tokens=20, stop_token_ids=[stop2]),
              3: SamplingParams(max_new_tokens=4), 4: SamplingParams(max_new_tokens=12),
              5: SamplingParams(max_new_tokens=30)}
    ids = {}

    def add(k):
        return lambda eng: ids.__setitem__(k, eng.add_request(prompts[k], params[k]))

    def script():
        return {0: lambda eng: [add(k)(eng) for k in (1, 2, 3)], 5: add(4), 9: add(5),
                16: lambda eng: eng.abort(ids[5])}

    results = {}
    for ahead in (False, True):
        ids.clear()
        eng = make_engine(ahead, pages=pages)
        trace = drive(eng, script())
        outs = {k: eng.collect(ids[k]) for k in sorted(ids)}
        eng.runner.alloc.check()
        assert eng.runner.alloc.free_pages() == pages and eng.runner.alloc.num_requests() == 0
        results[ahead] = (trace, {k: (o.token_ids, o.finish_reason) for k, o in outs.items()}, eng)
    base, with_ahead = results[False], results[True]
    assert with_ahead[0] == base[0] and with_ahead[1] == base[1]
    for k in (1, 2, 3, 4):
        want = expected_output(ids[k], prompts[k], params[k].max_new_tokens, params[k].stop_token_ids)
        assert base[1][k][0] == want
    assert base[1][2][1] == "stop_token" and base[1][5][1] == "cancelled" and base[1][1][1] == "max_tokens"
    eng = with_ahead[2]
    launched = [e for e in eng.runner.log if e[0] == "ahead"]
    assert base[2].steps_ahead == 0 and not [e for e in base[2].runner.log if e[0] == "ahead"]
    assert eng.steps_ahead >= 8 and len(launched) >= eng.steps_ahead      # some launches were dropped or partly used


def test_a_launched_step_is_dropped_when_a_request_arrives():
    eng = make_engine(True)
    a = eng.add_request([5, 6, 7], SamplingParams(max_new_tokens=10))
    eng.step()                                                   # the prompt
    eng.step()                                                   # first decode step; the next one is launched ahead
    assert eng._ahead is not None and eng.runner.log[-1] == ("ahead", (a,))
    b = eng.add_request([1, 2], SamplingParams(max_new_tokens=3))
    out = eng.step()                                             # the decision now holds a prompt: the launch is dropped
    assert eng.runner.log[-1][0] == "mixed" and eng.steps_ahead == 0
    assert sorted(r for r, _ in out) == [a, b]
    while eng.has_unfinished():
        eng.step()
    assert eng.collect(a).token_ids == expected_output(a, [5, 6, 7], 10)
    assert eng.collect(b).token_ids == expected_output(b, [1, 2], 3)
    eng.runner.alloc.check()


def test_nothing_is_launched_ahead_of_a_last_token():
    eng = make_engine(True)
    a = eng.add_request([5, 6, 7], SamplingParams(max_new_tokens=3))
    eng.step()                                                   # prompt -> token 1
    eng.step()                                                   # token 2; token 3 is the last: still launched ahead?
    assert eng._ahead is not None                                # yes: the step that makes token 3 is known
    eng.step()                                                   # token 3 ends the request: nothing follows it
    assert eng._ahead is None and not eng.has_unfinished()
    assert eng.collect(a).token_ids == expected_output(a, [5, 6, 7], 3)
    assert [e[0] for e in eng.runner.log] == ["mixed", "step", "ahead"]


def test_stream_yields_every_token_as_its_step_ends():
    """``Engine.stream``: one response per generated token, in step order, the last one of a request
    marked finished with its reason; afterwards the engine has forgotten the requests."""
    eng = make_engine(True)
    prompts = [[3, 4, 5], [9] * 7, [1]]
    stop = expected_output(2, prompts[1], 9)[4]
    params = [SamplingParams(max_new_tokens=6), SamplingParams(max_new_tokens=9, stop_token_ids=[stop]),
              SamplingParams(max_new_tokens=2)]
    got, last = {}, {}
    for r in eng.stream(prompts, params):
        assert r.request_id not in last, "a response after the finishing one"
        got.setdefault(r.request_id, []).append(r.token_id)
        if r.is_finished:
            last[r.request_id] = r.finish_reason
    assert got[1] == expected_output(1, prompts[0], 6) and last[1] == "max_tokens"
    assert got[2] == expected_output(2, prompts[1], 9, [stop]) and last[2] == "stop_token" and got[2][-1] == stop
    assert got[3] == expected_output(3, prompts[2], 2) and last[3] == "max_tokens"
    # the engine keeps nothing of a streamed request once its last response is out
    assert not eng.has_unfinished() and list(eng.scheduler.finished()) == []
    with pytest.raises(SchedulerError):
        eng.collect(2)
    eng.runner.alloc.check()


def test_requests_are_checked_when_they_are_added():
    from railgun_b200.engine.scheduler import SchedulerError
    eng = make_engine(False)
    for bad in ([1, 97], [-1, 2], [1.5, 2.0]):                       # outside the vocabulary of 97, or no integers
        with pytest.raises(ValueError, match="prompt token ids"):
            eng.add_request(bad)
    with pytest.raises(SchedulerError, match="empty"):
        eng.add_request([])
    with pytest.raises(SchedulerError, match="max_model_len"):
        eng.add_request([1] * 500, SamplingParams(max_new_tokens=100))
    with pytest.raises(ValueError):
        eng.add_request([1], SamplingParams(top_p=0.0))
    assert not eng.has_unfinished()
    rid = eng.add_request(np.array([3, 4, 5]), SamplingParams(max_new_tokens=2))      # arrays are taken as lists are
    while eng.has_unfinished():
        eng.step()
    assert eng.collect(rid).token_ids == expected_output(rid, [3, 4, 5], 2)
