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
    """The decode graphs read the rows' sampling parameters from the tail of the packed buffer: 64-bit seeds
    and draw counters first (at an even offset), then temperature, top-k, top-p; rows beyond the step's
    requests are greedy."""
    from railgun_b200.engine.runner import fill_sampling, sampling_views
    B, off = 4, 38
    buf = np.zeros(off + 7 * B, dtype=np.int32)
    views = sampling_views(buf, off, B)
    fill_sampling(views, dict(temperature=np.array([0.5, 0.0, 1.5], dtype=np.float32), top_k=np.array([3, 0, 40]),
                              top_p=np.array([0.75, 1.0, 0.25], dtype=np.float32),
                              seed=np.array([7, -1, 2 ** 62], dtype=np.int64), counter=np.array([0, 11, 12345678901])), 3)
    assert buf[off:off + 2 * B].view(np.int64).tolist() == [7, -1, 2 ** 62, 0]
    assert buf[off + 2 * B:off + 4 * B].view(np.int64).tolist() == [0, 11, 12345678901, 0]
    assert buf[off + 4 * B:off + 5 * B].view(np.float32).tolist() == [0.5, 0.0, 1.5, 0.0]
    assert buf[off + 5 * B:off + 6 * B].tolist() == [3, 0, 40, 0]
    assert buf[off + 6 * B:off + 7 * B].view(np.float32).tolist() == [0.75, 1.0, 0.25, 0.0]
    fill_sampling(views, None, 2)                               # a greedy step: every temperature is zero again
    assert not buf[off + 4 * B:off + 5 * B].any()
    assert not buf[:off].any()


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
