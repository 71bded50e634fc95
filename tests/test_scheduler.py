"""The scheduler's decisions, without a model: sampled tokens are fed by hand
(pattern of crates/vllm-scheduler/src/scheduler.rs:445-516 and
crates/vllm-scheduler/src/request.rs:210-248)."""
import numpy as np
import pytest

from railgun_b200.cache.manager import PageAllocator
from railgun_b200.engine.scheduler import Scheduler, SchedulerConfig, SchedulerError


def make(pages=32, page=4, seats=8, budget=64, chunk=0, max_len=256, window=0):
    a = PageAllocator([page], [pages], [window], seats)
    return a, Scheduler(a, SchedulerConfig(budget, seats, chunk, max_len))


def run_step(s, token_of=lambda rid, k: 1000 + k):
    es = s.schedule()
    ids = [e.request_id for e in es if e.want_last]
    s.update(ids, [token_of(r, s.num_generated(r)) for r in ids])
    return es


def test_prefill_then_decode_then_finish():
    a, s = make()
    s.add_request(1, [5, 6, 7, 8, 9], 3)
    es = s.schedule()
    assert [(e.request_id, e.start, e.tokens.tolist(), e.want_last) for e in es] == [(1, 0, [5, 6, 7, 8, 9], True)]
    assert s.num_running == 1 and s.num_waiting == 0
    s.update([1], [42])
    es = s.schedule()                                  # the sampled token is fed at the next position
    assert [(e.start, e.tokens.tolist(), e.want_last) for e in es] == [(5, [42], True)]
    s.update([1], [43])
    run_step(s, lambda r, k: 44)
    assert s.finished() == [1] and s.finish_reason(1) == "max_tokens" and s.outputs(1) == [42, 43, 44]
    assert s.num_running == 0 and a.free_pages() == 32 and a.num_requests() == 0
    a.check()


def test_three_requests_share_a_step():
    a, s = make()
    for i in range(3):
        s.add_request(i + 1, [1] * (3 + i), 2)
    es = s.schedule()
    assert [e.request_id for e in es] == [1, 2, 3] and sum(len(e.tokens) for e in es) == 12


def test_stop_token_is_kept_and_ends_the_request():
    a, s = make()
    s.add_request(1, [1, 2, 3], 10, stop_token_ids=[7, 9])
    run_step(s, lambda r, k: 5)
    run_step(s, lambda r, k: 9)
    assert s.finish_reason(1) == "stop_token" and s.outputs(1) == [5, 9]


def test_stop_wins_over_max_tokens():
    a, s = make()
    s.add_request(1, [1], 1, stop_token_ids=[3])
    run_step(s, lambda r, k: 3)
    assert s.finish_reason(1) == "stop_token"


def test_refusals():
    a, s = make(max_len=16)
    with pytest.raises(SchedulerError):
        s.add_request(1, [], 4)
    with pytest.raises(SchedulerError) as e:
        s.add_request(1, [1] * 10, 7)                   # 17 > max_model_len
    assert "max_model_len" in str(e.value)
    s.add_request(1, [1] * 10, 6)
    with pytest.raises(SchedulerError):
        s.add_request(1, [1], 1)
    with pytest.raises(SchedulerError):
        s.add_request(2, [1], 0)


def test_long_prompt_continues_under_the_token_budget():
    a, s = make(pages=64, budget=32)
    prompt = list(range(100))
    s.add_request(1, prompt, 2)
    seen, wants = [], []
    for _ in range(4):
        es = run_step(s)
        assert len(es) == 1
        seen += es[0].tokens.tolist()
        wants.append(es[0].want_last)
        assert es[0].start == len(seen) - len(es[0].tokens)
    assert seen == prompt and wants == [False, False, False, True]
    es = run_step(s)
    assert es[0].start == 100 and len(es[0].tokens) == 1


def test_max_prefill_chunk_and_decodes_first():
    a, s = make(pages=64, budget=40, chunk=16)
    s.add_request(1, [1] * 4, 8)
    run_step(s)                                         # request 1 is decoding from now on
    s.add_request(2, [2] * 40, 2)
    es = run_step(s)
    assert [(e.request_id, len(e.tokens)) for e in es] == [(1, 1), (2, 16)]
    es = run_step(s)
    assert [(e.request_id, len(e.tokens), e.want_last) for e in es] == [(1, 1, True), (2, 16, False)]
    es = run_step(s)
    assert [(e.request_id, len(e.tokens), e.want_last) for e in es] == [(1, 1, True), (2, 8, True)]


def test_budget_is_shared_and_admission_is_fifo():
    a, s = make(pages=64, budget=10)
    s.add_request(1, [1] * 6, 2)
    s.add_request(2, [2] * 6, 2)
    s.add_request(3, [3] * 2, 2)
    es = s.schedule()
    # request 2 gets what is left of the budget; request 3 waits behind it
    assert [(e.request_id, len(e.tokens), e.want_last) for e in es] == [(1, 6, True), (2, 4, False)]


def test_seats_limit():
    a, s = make(seats=2)
    for i in range(3):
        s.add_request(i + 1, [1, 2], 1)
    es = run_step(s)
    assert [e.request_id for e in es] == [1, 2] and s.num_waiting == 1
    es = run_step(s)
    assert [e.request_id for e in es] == [3]


def test_pages_run_out_newest_request_is_preempted_and_recomputed():
    a, s = make(pages=6, page=4, budget=64)
    s.add_request(1, [1] * 8, 12)                       # 2 pages, grows
    s.add_request(2, [2] * 7, 12)                       # 2 pages, grows
    tok = lambda r, k: 100 * r + k
    run_step(s, tok)                                    # both prefilled: 4 pages held
    steps = 0
    preempted_seen = False
    while not (s.finish_reason(1) and s.finish_reason(2)):
        es = run_step(s, tok)
        if s.preempted():
            preempted_seen = True
            assert s.preempted() == [2]                 # the most recently admitted gives way
        for e in es:
            assert e.start == 0 or len(e.tokens) == 1 or e.request_id == 2
        a.check()
        steps += 1
        assert steps < 100
    assert preempted_seen and s.num_preemptions(2) >= 1 and s.num_preemptions(1) == 0
    # generated tokens survive preemption: the sequence is what an undisturbed run gives
    assert s.outputs(1) == [100 + k for k in range(12)]
    assert s.outputs(2) == [200 + k for k in range(12)]
    assert a.free_pages() == 6


def test_preempted_request_is_recomputed_as_one_prompt():
    a, s = make(pages=5, page=4, budget=64)
    s.add_request(1, [1] * 6, 8)
    s.add_request(2, [2] * 6, 8)                        # admitted: 2 pages and one to spare
    assert len(run_step(s)) == 2                        # 2 + 2 pages held
    run_step(s)
    run_step(s)
    es = run_step(s)                                    # position 8 of each needs a third page; one is left
    assert s.preempted() == [2] and [e.request_id for e in es] == [1]
    assert s.num_waiting == 1 and not a.has(2)
    while s.finish_reason(1) is None:
        es = run_step(s)
        assert [e.request_id for e in es] == [1]        # nothing is admitted while request 1 needs the room
    es = s.schedule()                                   # request 2 comes back: prompt + its 3 tokens, from 0
    assert [(e.request_id, e.start, len(e.tokens), e.want_last) for e in es] == [(2, 0, 9, True)]
    assert es[0].tokens.tolist() == [2] * 6 + [1000, 1001, 1002]


def test_request_that_cannot_fit_alone_ends_with_an_error():
    a, s = make(pages=2, page=4)
    s.add_request(1, [1] * 9, 2)                        # needs 3 pages for its prompt
    s.add_request(2, [1] * 3, 2)
    es = s.schedule()
    assert s.finish_reason(1) == "error" and "out of KV cache blocks" in s.error(1)
    assert [e.request_id for e in es] == [2]
    # one that fits at first and outgrows the pool
    a, s = make(pages=2, page=4)
    s.add_request(1, [1] * 7, 8)
    for _ in range(3):
        run_step(s)
    assert s.finish_reason(1) == "error" and s.outputs(1) == [1000, 1001]
    assert a.free_pages() == 2 and a.num_requests() == 0


def test_abort_waiting_and_running():
    a, s = make(seats=1)
    s.add_request(1, [1, 2, 3], 5)
    s.add_request(2, [1, 2, 3], 5)
    run_step(s)
    s.abort(2)
    assert s.finish_reason(2) == "cancelled" and s.num_waiting == 0
    s.abort(1)
    assert s.finish_reason(1) == "cancelled" and s.num_running == 0 and a.free_pages() == 32
    with pytest.raises(SchedulerError):
        s.abort(77)
    s.forget(1)
    with pytest.raises(SchedulerError):
        s.finish_reason(1)


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_with_undisturbed_outputs(seed):
    rng = np.random.default_rng(seed)
    a, s = make(pages=40, page=4, seats=5, budget=48, chunk=int(rng.choice([0, 8, 20])), max_len=200)
    want = {}
    pending = [(rid, list(rng.integers(0, 50, size=int(rng.integers(1, 60)))), int(rng.integers(1, 25)))
               for rid in range(1, 25)]
    tok = lambda r, k: (r * 31 + k * 7) % 50
    steps = 0
    while pending or s.num_waiting or s.num_running:
        while pending and rng.random() < 0.5:
            rid, prompt, n_new = pending.pop(0)
            s.add_request(rid, prompt, n_new)
            want[rid] = [tok(rid, k) for k in range(n_new)]
        es = s.schedule()
        assert sum(len(e.tokens) for e in es) <= 48
        assert len({e.request_id for e in es}) == len(es)
        for e in es:
            assert e.start == a.num_computed(e.request_id)
            assert len(a.block_table(e.request_id)) * 4 >= e.start + len(e.tokens)
        ids = [e.request_id for e in es if e.want_last]
        s.update(ids, [tok(r, s.num_generated(r)) for r in ids])
        a.check()
        steps += 1
        assert steps < 5000
    assert sorted(s.finished()) == sorted(want)
    for rid, toks in want.items():
        assert s.finish_reason(rid) == "max_tokens" and s.outputs(rid) == toks
    assert a.free_pages() == 40 and a.free_slots() == 5


def test_when_the_next_decision_is_known_ahead():
    """The engine launches the next decode step early only when the scheduler says that its decision is
    known: all running requests decode, none can end by length, nothing was preempted."""
    a, s = make(pages=8, page=4, seats=2)
    s.add_request(1, [1, 2, 3], 4)
    s.add_request(2, [4, 5], 3)
    s.add_request(3, [6, 7, 8], 5)                     # no seat: waits
    es = s.schedule()
    assert [e.request_id for e in es] == [1, 2] and not s.next_step_predictable()     # prompts in the step
    s.update([1, 2], [10, 20])
    s.schedule()
    assert s.num_waiting == 1 and s.next_step_predictable()      # both decode; request 3 was refused a seat
    s.update([1, 2], [11, 21])
    s.schedule()
    assert not s.next_step_predictable()               # request 2 generates its last token in this step
    s.update([1, 2], [12, 22])
    es = s.schedule()                                  # request 2 is gone, request 3 takes its seat: a prompt
    assert sorted(e.request_id for e in es) == [1, 3] and not s.next_step_predictable()
    assert s.num_generated_many(np.array([1, 3])).tolist() == [3, 0]
    s.update([1, 3], [13, 30])
    assert s.finished() == [2, 1]
    s.schedule()
    assert s.next_step_predictable()                   # request 3 decodes alone
    # a preemption in the decision: nothing is launched ahead
    a2, s2 = make(pages=3, page=4, seats=4)
    s2.add_request(1, [1] * 4, 8)
    s2.add_request(2, [2] * 4, 8)
    run_step(s2)
    while not s2.preempted():
        assert s2.num_running == 2
        es = s2.schedule()
        if s2.preempted():
            assert not s2.next_step_predictable()
            break
        s2.update([e.request_id for e in es], [7] * len(es))
