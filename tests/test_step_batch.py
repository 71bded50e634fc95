"""Packing of a step (engine/batch.py over the C++ cache manager), on the CPU:
every field against a construction written out here with numpy, and the errors
that must leave the cache's bookkeeping as it was."""
import numpy as np
import pytest

from railgun_b200.cache.manager import OutOfPages, PageAllocator
from railgun_b200.engine.batch import BatchError, StepEntry, build_step_batch

VOCAB, MAX_POS = 1000, 4096


def expected_fields(entries, starts, tables, slots, page_sizes):
    """The step's fields from first principles: one loop per token."""
    tok, pos, req, want_rows, cu, tiles, tiles128, dec = [], [], [], [], [0], [], [], []
    slot_maps = [[] for _ in page_sizes]
    for i, e in enumerate(entries):
        off = len(tok)
        for k, t in enumerate(e.tokens):
            tok.append(int(t)), pos.append(starts[i] + k), req.append(i)
            for g, ps in enumerate(page_sizes):
                p = starts[i] + k
                slot_maps[g].append(max(tables[g][i][p // ps], 0) * ps + p % ps)
        want_rows += [off + w for w in e.want]
        cu.append(len(tok))
        n = len(e.tokens)
        if n == 1:
            dec.append(off)
        else:
            tiles += [(off + k, min(64, n - k), i) for k in range(0, n, 64)]
            tiles128 += [(off + k, min(128, n - k), i) for k in range(0, n, 128)]
    return dict(tok=tok, pos=pos, req=req, want_rows=want_rows, cu=cu, tiles=tiles, tiles128=tiles128, dec=dec,
                slot_maps=slot_maps, ctx=[starts[i] + len(e.tokens) for i, e in enumerate(entries)], slots=slots)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_fields_of_random_steps(seed):
    rng = np.random.default_rng(seed)
    page_sizes, windows = [8, 16], [0, 40]                  # the second group gives pages back behind a window
    alloc = PageAllocator(page_sizes, [400, 200], windows, 8)
    live = {}
    for step in range(12):
        ids = [int(i) for i in rng.choice(6, size=int(rng.integers(1, 5)), replace=False)]
        entries = []
        for rid in ids:
            n = int(rng.choice([1, 1, 2, 3, 17, 64, 65, 130, 200]))
            toks = rng.integers(0, VOCAB, size=n)
            toks = toks.tolist() if rng.random() < 0.5 else toks        # lists and arrays are both taken
            want = sorted(int(w) for w in rng.choice(n, size=int(rng.integers(0, min(n, 3) + 1)), replace=False))
            entries.append(StepEntry(rid, toks, want))
        starts = [live.get(rid, 0) for rid in ids]
        b = build_step_batch(entries, alloc, page_sizes, VOCAB, MAX_POS, "cpu")
        tables = [[alloc.block_table(rid, g) for rid in ids] for g in range(2)]
        exp = expected_fields(entries, starts, tables, [alloc.slot(rid) for rid in ids], page_sizes)
        assert b.token_ids.tolist() == exp["tok"] and b.positions.tolist() == exp["pos"]
        assert b.req_of_token.tolist() == exp["req"] and b.want_rows.tolist() == exp["want_rows"]
        assert b.cu_seqlens.tolist() == exp["cu"] and b.context_lens.tolist() == exp["ctx"]
        assert b.start_pos.tolist() == starts and b.state_slots.tolist() == exp["slots"]
        assert list(b.host_cu_seqlens) == exp["cu"] and list(b.host_start_pos) == starts
        assert list(b.host_state_slots) == exp["slots"]
        assert b.host_request_ids.tolist() == ids and b.host_context_lens.tolist() == exp["ctx"]
        for g in range(2):
            assert b.slot_mapping[g].tolist() == exp["slot_maps"][g]
            width = b.block_table[g].shape[1]
            longest = max(len(t) for t in tables[g])
            assert width >= longest and width & (width - 1) == 0 and width < 2 * max(longest, 1)
            for i, t in enumerate(tables[g]):
                row = b.block_table[g][i].tolist()
                assert row[:len(t)] == [max(int(p), 0) for p in t] and not any(row[len(t):])
        got_tiles = b.prefill_tiles.tolist() if b.prefill_tiles is not None else []
        got_tiles128 = b.prefill_tiles128.tolist() if b.prefill_tiles128 is not None else []
        assert [tuple(t) for t in got_tiles] == exp["tiles"] and b.num_prefill_tiles == len(exp["tiles"])
        assert [tuple(t) for t in got_tiles128] == exp["tiles128"] and b.num_prefill_tiles128 == len(exp["tiles128"])
        assert (b.decode_rows.tolist() if b.decode_rows is not None else []) == exp["dec"]
        assert b.num_tokens == len(exp["tok"]) and b.num_wanted == len(exp["want_rows"])
        assert b.max_query_len == max(len(e.tokens) for e in entries) and b.max_context_len == max(exp["ctx"])
        assert b.decode_only == all(len(e.tokens) == 1 for e in entries)
        assert b.layout == (tuple(len(e.tokens) for e in entries), len(exp["want_rows"]),
                            tuple(t.shape[1] for t in b.block_table))
        alloc.commit_many(b.host_request_ids, b.host_context_lens)
        for e, s in zip(entries, starts):
            assert alloc.num_computed(e.request_id) == s + len(e.tokens)
            live[e.request_id] = s + len(e.tokens)
        for rid in ids:
            if live[rid] > 300 or rng.random() < 0.2:
                alloc.release(rid)
                del live[rid]
        alloc.check()


def test_a_bad_step_changes_nothing():
    alloc = PageAllocator([16], [8], [0], 4)
    build = lambda entries, max_pos=MAX_POS: build_step_batch(entries, alloc, [16], VOCAB, max_pos, "cpu")
    build([StepEntry(1, [5, 6, 7], [2])])
    alloc.commit(1, 3)
    before = (alloc.num_requests(), alloc.free_pages(), alloc.free_slots())
    cases = [
        ([], "at least one entry"),
        ([StepEntry(2, [1, 2]), StepEntry(2, [3])], "request 2 appears twice"),
        ([StepEntry(2, [])], "request 2: an entry needs at least one token"),
        ([StepEntry(2, [1, VOCAB])], r"request 2: token ids must be in \[0, 1000\)"),
        ([StepEntry(2, [-1])], "request 2: token ids must be in"),
        ([StepEntry(2, [1.5, 2.0])], "request 2: token ids must be in"),
        ([StepEntry(3, [1, 2]), StepEntry(2, [1, 2, 3], [3])], "request 2: wanted place 3 is outside its 3 tokens"),
        ([StepEntry(2, [1, 2, 3], [-1])], "request 2: wanted place -1 is outside"),
    ]
    for entries, message in cases:
        with pytest.raises(BatchError, match=message):
            build(entries)
        assert (alloc.num_requests(), alloc.free_pages(), alloc.free_slots()) == before
    with pytest.raises(BatchError, match="request 1: position 20 is beyond the model's max_position_embeddings 20"):
        build([StepEntry(3, [1]), StepEntry(1, list(range(18)))], max_pos=20)
    assert (alloc.num_requests(), alloc.free_pages(), alloc.free_slots()) == before
    alloc.check()


def test_a_step_that_runs_out_of_pages_gives_back_the_requests_it_added():
    alloc = PageAllocator([16], [4], [0], 4)
    build_step_batch([StepEntry(1, list(range(20)))], alloc, [16], VOCAB, MAX_POS, "cpu")
    alloc.commit(1, 20)
    with pytest.raises(OutOfPages):
        build_step_batch([StepEntry(2, list(range(16))), StepEntry(3, list(range(40)))], alloc, [16], VOCAB, MAX_POS,
                         "cpu")
    assert not alloc.has(2) and not alloc.has(3) and alloc.has(1)
    assert alloc.free_pages() == 2 and alloc.free_slots() == 3
    alloc.check()
    # and without a free state slot
    small = PageAllocator([16], [8], [0], 1)
    build_step_batch([StepEntry(1, [1])], small, [16], VOCAB, MAX_POS, "cpu")
    with pytest.raises(Exception, match="out of state slots"):
        build_step_batch([StepEntry(2, [1])], small, [16], VOCAB, MAX_POS, "cpu")
    assert small.num_requests() == 1
    small.check()


def test_sampling_parameters_in_the_packed_decode_buffer():
    """The decode graphs read the rows' sampling parameters from the tail of the packed buffer, where the
    cache manager writes them from the requests' slot records: 64-bit seeds and draw counters first, then
    temperature, top-k, top-p; rows beyond the step's requests are greedy."""
    from railgun_b200.engine.runner import sampling_views
    alloc = PageAllocator([16], [16], [0], 8)
    for rid in (5, 6, 7):
        alloc.add_request(rid)
        alloc.reserve(rid, 3)
        alloc.commit(rid, 3)
    alloc.set_request(5, prompt_len=3, num_generated=0, max_new_tokens=9, temperature=0.5, top_k=3, top_p=0.75, seed=7)
    alloc.set_request(7, prompt_len=1, num_generated=2, max_new_tokens=9, temperature=1.5, top_k=40, top_p=0.25,
                      seed=2 ** 64 - 1)
    B, MB = 4, 2
    off = (5 + 1) * B + B * MB                               # what StaticDecodeBatch computes for one group (even)
    buf = np.full(off + 7 * B, -99, dtype=np.int32)
    ids = np.array([5, 6, 7], dtype=np.int64)
    assert alloc.pack_decode(ids, B, MB, buf[B:], sampling=buf[off:], draw_ahead=0) is True
    v = sampling_views(buf, off, B)
    assert v["seed"].tolist() == [7, 0, -1, 0] and v["counter"].tolist() == [0, 0, 2, 0]
    assert v["temperature"].tolist() == [0.5, 0.0, 1.5, 0.0] and v["top_k"].tolist() == [3, 0, 40, 0]
    assert v["top_p"].tolist() == [0.75, 1.0, 0.25, 1.0]
    assert buf[B:2 * B].tolist() == [3, 3, 3, 0]              # positions; the padding row is at 0
    # the step after it, launched ahead: the draws are numbered one further
    alloc.pack_decode(ids, B, MB, buf[B:], ahead=1, sampling=buf[off:], draw_ahead=1)
    assert v["counter"].tolist() == [1, 1, 3, 0] and buf[B:2 * B].tolist() == [4, 4, 4, 0]
    # all greedy: nothing samples
    assert alloc.pack_decode(np.array([6], dtype=np.int64), B, MB, buf[B:], sampling=buf[off:]) is False
    assert not v["temperature"].any()


def test_request_records():
    """One record of fixed size per state slot: the cache manager keeps the position, the scheduler the lengths
    and the sampling parameters; a slot's record is cleared when the request leaves, and the scheduler writes it
    again when a preempted request comes back."""
    from railgun_b200.cache.manager import REQUEST_RECORD
    from railgun_b200.engine.scheduler import Scheduler, SchedulerConfig
    alloc = PageAllocator([4], [6], [0], 2)
    assert REQUEST_RECORD.itemsize == 64 and alloc.records.shape == (2,)
    assert alloc.records["request_id"].tolist() == [-1, -1]
    s = Scheduler(alloc, SchedulerConfig(64, 2, 0, 64))
    s.add_request(11, [1] * 7, 9, temperature=0.7, top_k=5, top_p=0.9, seed=2 ** 63 + 5)
    s.add_request(12, [2] * 6, 9)
    s.schedule()
    r = alloc.record(11)
    assert (r["request_id"], r["num_computed"], r["prompt_len"], r["num_generated"], r["max_new_tokens"]) == (11, 0, 7, 0, 9)
    assert (float(r["temperature"]), r["top_k"], float(r["top_p"]), int(r["seed"])) == (np.float32(0.7), 5, np.float32(0.9), 2 ** 63 + 5)
    s.update([11, 12], [40, 41])
    r = alloc.record(11)
    assert (r["num_computed"], r["num_generated"], r["last_token"]) == (7, 1, 40)
    assert s.sampling_many([11, 12])["counter"].tolist() == [1, 1]
    # decoding until the pool is exhausted preempts the request admitted last; its record goes with its slot
    for step in range(6):
        entries = s.schedule()
        if s.preempted():
            break
        s.update([e.request_id for e in entries], [50 + step] * len(entries))
    assert s.preempted() == [12] and not alloc.has(12)
    assert sorted(alloc.records["request_id"].tolist()) == [-1, 11]
    generated = s.num_generated(12)
    s.abort(11)
    s.schedule()                                             # 12 comes back, as one longer prompt
    r = alloc.record(12)
    assert (r["prompt_len"], r["num_generated"], r["num_computed"]) == (6, generated, 0) and r["temperature"] == 0.0
    alloc.check()


def test_rows_of_a_step_launched_ahead():
    """Which rows of a launched step answer a decision: all of them in order, a subset (requests that ended
    are skipped), or none if the decision names a request the step did not hold."""
    from types import SimpleNamespace
    from railgun_b200.engine.engine import Engine
    launched = SimpleNamespace(ids=np.array([4, 9, 2, 7], dtype=np.int64))
    rows = Engine._rows_of_launched(launched, np.array([4, 9, 2, 7], dtype=np.int64))
    assert rows == slice(0, 4)
    assert Engine._rows_of_launched(launched, np.array([4, 2, 7], dtype=np.int64)).tolist() == [0, 2, 3]
    assert Engine._rows_of_launched(launched, np.array([7, 4], dtype=np.int64)).tolist() == [3, 0]
    assert Engine._rows_of_launched(launched, np.array([4, 9, 2, 5], dtype=np.int64)) is None
