"""Generation through the Python entry point and the command line: greedy
against the plain implementation, seeded temperature sampling, preemption,
long decoding and the first tokens of a sequence."""
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def assert_greedy_consistent(plain, prompt, out, tol):
    """Teacher-forced: every generated token's plain logit is the row's
    maximum, up to ``tol`` of the largest absolute logit."""
    logits = plain.forward(list(prompt) + list(out))
    for i, t in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert row[t] >= row.max() - tol * np.abs(logits).max(), f"generated token {i} ({t}) is not the argmax"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(name, dtype):
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY[name]
    lengths = [5, 17, 33] if name == "A" else [1, 9, 40, 63, 100]
    n_new = 8 if name == "A" else 12
    prompts = helpers.prompts(cfg["vocab_size"], lengths, seed=1 if name == "A" else 3)
    plain = P.PlainLlama(helpers.model_dir(name))
    eng = Engine(helpers.model_dir(name), dtype=dtype, block_size=page, num_gpu_blocks=64, max_num_seqs=8,
                 max_num_batched_tokens=64, max_prefill_chunk=32 if name == "B" else 0, max_model_len=256)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=n_new))
    exact = 0
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "max_tokens" and len(o.token_ids) == n_new
        assert_greedy_consistent(plain, p, o.token_ids, 1e-4 if dtype == "float32" else 6e-2)
        exact += int(o.token_ids == plain.greedy(p, n_new))
    assert exact >= (len(prompts) if dtype == "float32" else 1)
    assert eng.stats()["num_free_blocks"] == 64 and not eng.has_unfinished()


def test_first_tokens_of_a_sequence():
    """Prompts of one and two tokens, and the first generated tokens, in one batch."""
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY["A"]
    plain = P.PlainLlama(helpers.model_dir("A"))
    eng = Engine(helpers.model_dir("A"), dtype="float32", block_size=page, num_gpu_blocks=32, max_num_seqs=8)
    prompts = [[7], [200, 3], [0], [255, 255, 255]]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=3))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy(p, 3)


def test_long_decoding_and_stop_token():
    """A short prompt decoded for 200 tokens, token by token, across many pages."""
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY["B"]
    plain = P.PlainLlama(helpers.model_dir("B"))
    prompt = helpers.prompts(cfg["vocab_size"], [6], seed=12)[0]
    eng = Engine(helpers.model_dir("B"), dtype="float32", block_size=page, num_gpu_blocks=40, max_num_seqs=2,
                 max_model_len=512)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=200))[0]
    assert len(out.token_ids) == 200
    # teacher-forced check: every generated token is the plain argmax given the tokens before it
    logits = plain.forward(prompt + out.token_ids)
    for i, t in enumerate(out.token_ids):
        row = logits[len(prompt) - 1 + i]
        assert row[t] >= np.sort(row)[-1] - 1e-4 * np.abs(row).max(), f"generated token {i} is not the argmax"
    # the same request with a stop token ends there, stop token kept
    stop = out.token_ids[20]
    first = out.token_ids.index(stop)
    again = eng.generate([prompt], SamplingParams(max_new_tokens=200, stop_token_ids=[stop]))[0]
    assert again.finish_reason == "stop_token" and again.token_ids == out.token_ids[:first + 1]


def test_temperature_sampling_is_seeded_and_batch_invariant():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY["B"]
    prompts = helpers.prompts(cfg["vocab_size"], [9, 40, 63, 20], seed=3)
    params = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=100 + i) if i % 2 else
              SamplingParams(max_new_tokens=12) for i in range(4)]
    mk = lambda: Engine(helpers.model_dir("B"), dtype="float32", block_size=page, num_gpu_blocks=64, max_num_seqs=8,
                        max_prefill_chunk=32)
    together = mk().generate(prompts, params)
    eng = mk()
    alone = [eng.generate([p], sp)[0] for p, sp in zip(prompts, params)]
    for a, b in zip(together, alone):
        assert a.token_ids == b.token_ids
    other_seed = mk().generate([prompts[1]], SamplingParams(max_new_tokens=12, temperature=0.8, seed=999))[0]
    assert other_seed.token_ids != together[1].token_ids
    # each sampled token is what the plain sampler draws from the plain logits with the same seed and counter
    plain = P.PlainLlama(helpers.model_dir("B"))
    ids = list(prompts[1])
    for k, t in enumerate(together[1].token_ids):
        row = plain.forward(ids)[-1]
        p = P.filtered_probs(row, 0.8)
        c = np.cumsum(p)
        u = P.uniform_from_counter(101, k)
        assert c[t] - p[t] - 1e-4 <= u <= c[t] + 1e-4
        ids.append(t)


def test_preemption_does_not_change_the_outputs():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY["A"]
    prompts = helpers.prompts(cfg["vocab_size"], [30, 28, 25], seed=17)
    params = [SamplingParams(max_new_tokens=40, temperature=0.7 if i == 1 else 0.0, seed=5) for i in range(3)]
    roomy = Engine(helpers.model_dir("A"), dtype="float32", block_size=page, num_gpu_blocks=64, max_num_seqs=4,
                   max_model_len=256).generate(prompts, params)
    tight_engine = Engine(helpers.model_dir("A"), dtype="float32", block_size=page, num_gpu_blocks=9, max_num_seqs=4,
                          max_model_len=256)
    tight = tight_engine.generate(prompts, params)
    assert sum(o.num_preemptions for o in tight) >= 1 and sum(o.num_preemptions for o in roomy) == 0
    for a, b in zip(roomy, tight):
        assert a.token_ids == b.token_ids and b.finish_reason == "max_tokens"
    tight_engine.runner.alloc.check()
    # a request that cannot fit the pool even alone ends with an error, the others go on
    eng = Engine(helpers.model_dir("A"), dtype="float32", block_size=page, num_gpu_blocks=3, max_num_seqs=4,
                 max_model_len=256)
    outs = eng.generate([prompts[0], [1, 2, 3] * 20], SamplingParams(max_new_tokens=4))
    assert outs[0].finish_reason == "max_tokens"
    assert outs[1].finish_reason == "error" and "out of KV cache blocks" in outs[1].error


@pytest.mark.parametrize("sampled", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(dtype, sampled):
    """Decode steps are launched before the tokens of the step before are read.
    Requests that end at different lengths and on stop tokens, a request added
    in the middle, a request aborted in the middle and few pages (preemption):
    the outputs equal those of an engine that launches nothing ahead, step by
    step, and steps were indeed taken from launches made ahead."""
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY["B"]
    prompts = helpers.prompts(cfg["vocab_size"], [9, 40, 3, 63, 20], seed=21)
    plain = P.PlainLlama(helpers.model_dir("B"))
    stop = plain.greedy(prompts[1], 12)[7]               # ends request 1 in the middle of the others' decoding
    params = [SamplingParams(max_new_tokens=n, stop_token_ids=st, **more)
              for n, st, more in ((30, [], {}), (40, [stop], {}), (5, [], {}), (17, [], {}), (25, [], {}))]
    if sampled:                                          # some requests draw their tokens: the graph samples
        params[0] = SamplingParams(max_new_tokens=30, temperature=0.8, seed=3)
        params[3] = SamplingParams(max_new_tokens=17, temperature=1.1, top_k=20, top_p=0.9, seed=9)

    def run(ahead, blocks):
        eng = Engine(helpers.model_dir("B"), dtype=dtype, block_size=page, num_gpu_blocks=blocks, max_num_seqs=4,
                     max_num_batched_tokens=64, max_model_len=256)
        eng.run_ahead = ahead
        rids = [eng.add_request(p, sp) for p, sp in zip(prompts[:3], params[:3])]
        trace, steps = [], 0
        while eng.has_unfinished():
            out = eng.step()
            trace.append(sorted(out) if out else out)
            steps += 1
            if steps == 6:
                rids.append(eng.add_request(prompts[3], params[3]))     # arrives while the others decode
            if steps == 9:
                rids.append(eng.add_request(prompts[4], params[4]))
            if steps == 14:
                eng.abort(rids[4])
            assert steps < 400
        outs = [eng.collect(r) for r in rids]
        eng.runner.alloc.check()
        assert eng.stats()["num_free_blocks"] == blocks
        return outs, trace, eng.steps_ahead

    for blocks in (64, 22):
        base, base_trace, none_ahead = run(False, blocks)
        outs, trace, taken_ahead = run(True, blocks)
        assert none_ahead == 0 and taken_ahead > 10
        assert trace == base_trace
        for a, b in zip(outs, base):
            assert a.token_ids == b.token_ids and a.finish_reason == b.finish_reason
    assert base[1].finish_reason == "stop_token" and base[4].finish_reason == "cancelled"
    assert sampled or dtype == "bfloat16" or base[0].token_ids == plain.greedy(prompts[0], 30)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_many_live_requests(name, dtype):
    """Forty-eight requests, up to 64 seats (the reference's default is 256,
    crates/vllm-scheduler/src/scheduler.rs:47-58): decode steps of 17 to 48 rows
    take the library products, SiLU-mul on interleaved storage, the larger batch
    buckets and steps launched ahead at those sizes.  Greedy and sampled
    requests, prompts of mixed length cut into portions beside decoding
    requests, and a pool small enough that requests are preempted.  Every token
    is checked against the plain implementation, teacher-forced; in 32-bit the
    outputs also equal those of the same requests run one at a time."""
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY[name]
    rng = np.random.default_rng(31)
    lengths = [int(n) for n in rng.integers(2, 70, size=48)]
    prompts = helpers.prompts(cfg["vocab_size"], lengths, seed=32)
    params = []
    for i in range(48):
        n_new = int(rng.integers(6, 24))
        if i % 3 == 1:
            params.append(SamplingParams(max_new_tokens=n_new, temperature=0.8, seed=1000 + i))
        elif i % 3 == 2:
            params.append(SamplingParams(max_new_tokens=n_new, temperature=1.0, top_k=12, top_p=0.9, seed=2000 + i))
        else:
            params.append(SamplingParams(max_new_tokens=n_new))
    blocks = int(0.8 * sum(-(-n // page) for n in lengths))        # four fifths of what the prompts alone need
    eng = Engine(helpers.model_dir(name), dtype=dtype, block_size=page, num_gpu_blocks=blocks, max_num_seqs=64,
                 max_num_batched_tokens=256, max_model_len=128)
    widest = 0
    rids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
    while eng.has_unfinished():
        made = eng.step()
        widest = max(widest, len(made or ()))
    outs = [eng.collect(r) for r in rids]
    assert widest > 32, f"at most {widest} requests were live in a step"
    assert sum(o.num_preemptions for o in outs) >= 1
    eng.runner.alloc.check()
    assert eng.stats()["num_free_blocks"] == blocks
    plain = P.PlainLlama(helpers.model_dir(name))
    tol = 1e-4 if dtype == "float32" else 6e-2
    for p, sp, o in zip(prompts, params, outs):
        assert o.finish_reason == "max_tokens" and len(o.token_ids) == sp.max_new_tokens
        logits = plain.forward(list(p) + o.token_ids)
        for k, t in enumerate(o.token_ids):
            row = logits[len(p) - 1 + k]
            if sp.temperature == 0.0:
                assert row[t] >= row.max() - tol * np.abs(logits).max(), f"token {k} ({t}) is not the argmax"
            else:
                if dtype == "float32":
                    # the drawn token's interval of the plain distribution holds the draw's uniform number
                    pr = P.filtered_probs(row, sp.temperature, sp.top_k, sp.top_p)
                    c = np.cumsum(pr)
                    u = P.uniform_from_counter(sp.seed, k)
                    assert c[t] - pr[t] - 1e-4 <= u <= c[t] + 1e-4, f"token {k} ({t}) is not the plain draw"
                else:
                    # bfloat16 logits move every probability by several per cent, and with them the intervals;
                    # what must hold is that the token passes the plain filters (taken a little wider)
                    pr = P.filtered_probs(row, sp.temperature, sp.top_k + 3 if sp.top_k else 0, min(1.0, sp.top_p + 0.07))
                    assert pr[t] > 0.0, f"token {k} ({t}) is outside the plain top-k / top-p set"
    if dtype == "float32":
        one = Engine(helpers.model_dir(name), dtype=dtype, block_size=page, num_gpu_blocks=64, max_num_seqs=1,
                     max_model_len=128)
        for p, sp, o in list(zip(prompts, params, outs))[::5]:
            assert one.generate([p], sp)[0].token_ids == o.token_ids


def test_stream_gives_the_tokens_of_generate():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = helpers.TINY["A"]
    prompts = helpers.prompts(cfg["vocab_size"], [5, 17, 33], seed=1)
    params = [SamplingParams(max_new_tokens=n, temperature=t, seed=2) for n, t in ((8, 0.0), (3, 0.9), (12, 0.0))]
    kw = dict(dtype="float32", block_size=page, num_gpu_blocks=64, max_num_seqs=8)
    outs = Engine(helpers.model_dir("A"), **kw).generate(prompts, params)
    got, reasons = {}, {}
    for r in Engine(helpers.model_dir("A"), **kw).stream(prompts, params):
        got.setdefault(r.request_id, []).append(r.token_id)
        if r.is_finished:
            reasons[r.request_id] = r.finish_reason
    assert [got[o.request_id] for o in outs] == [o.token_ids for o in outs]
    assert [reasons[o.request_id] for o in outs] == [o.finish_reason for o in outs] == ["max_tokens"] * 3


def test_engine_refuses_bad_requests():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    from railgun_b200.engine.scheduler import SchedulerError
    eng = Engine(helpers.model_dir("A"), dtype="float32", num_gpu_blocks=16, max_model_len=64)
    with pytest.raises(ValueError):
        eng.add_request([1, 256])                         # id outside the vocabulary
    with pytest.raises(SchedulerError):
        eng.add_request([1] * 60, SamplingParams(max_new_tokens=10))
    with pytest.raises(ValueError):
        eng.add_request([1], SamplingParams(temperature=-1.0))


def test_generate_command(tmp_path):
    cfg, _, page = helpers.TINY["A"]
    plain = P.PlainLlama(helpers.model_dir("A"))
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "railgun"), "generate", "--model", str(helpers.model_dir("A")),
         "--prompt-ids", "5,6,7;100,2", "--max-tokens", "6", "--dtype", "f32", "--show-token-ids",
         "--num-gpu-blocks", "32"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = proc.stdout.strip().splitlines()
    assert lines[0] == "prompt ids: [5, 6, 7]"
    assert lines[1] == ",".join(map(str, plain.greedy([5, 6, 7], 6)))
    assert lines[3] == ",".join(map(str, plain.greedy([100, 2], 6)))
    assert lines[-1].startswith("[stats] 12 tokens") and "tok/s" in lines[-1]


def test_generate_command_with_random_weights(tmp_path):
    """``--random-weights SEED``: the folder's config.json with weights drawn from the seed; the same seed gives
    the same tokens, another seed other weights (the configuration with an untied head: with a tied one and small
    random weights every model just repeats its last token)."""
    def run(seed):
        proc = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "railgun"), "generate", "--model", str(helpers.model_dir("B")),
             "--prompt-ids", "5,6,7", "--max-tokens", "8", "--dtype", "f32", "--num-gpu-blocks", "32",
             "--random-weights", str(seed)], capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        return proc.stdout.strip().splitlines()[0]
    first = run(3)
    assert len(first.split(",")) == 8 and run(3) == first and run(4) != first


def test_generate_command_with_a_text_prompt(tmp_path):
    """``--prompt/-p TEXT`` with a tokenizer.json in the model folder (a word-level toy made here): the
    same tokens as the ids path, the text printed after the prompt, generation ended by the tokenizer's
    end-of-sequence token."""
    import shutil
    from tokenizers import Tokenizer, models, pre_tokenizers
    cfg, _, page = helpers.TINY["A"]
    plain = P.PlainLlama(helpers.model_dir("A"))
    mdir = tmp_path / "with_tokenizer"
    shutil.copytree(helpers.model_dir("A"), mdir)
    ref = plain.greedy([5, 6, 7], 6)
    eos = ref[3]                                                 # the fourth generated token ends the text
    vocab = {f"w{i}": i for i in range(cfg["vocab_size"])}
    del vocab[f"w{eos}"]
    vocab["</s>"] = eos
    tok = Tokenizer(models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "railgun"), "generate", "-m", str(mdir), "-p", "w5 w6 w7",
         "--max-tokens", "6", "--dtype", "f32", "--show-token-ids", "--num-gpu-blocks", "32"],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = proc.stdout.strip().splitlines()
    first = ref[:ref.index(eos) + 1]                             # the stop token is kept, as in the engine path
    assert lines[0] == "prompt ids: [5, 6, 7]"
    assert lines[1].startswith("w5 w6 w7") and f"w{first[0]}" in lines[1]
    assert lines[2] == ",".join(map(str, first))
    # without a tokenizer the option is refused before anything is loaded
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "railgun"), "generate", "-m", str(helpers.model_dir("A")), "-p", "w5"],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 2 and "tokenizer.json does not exist" in proc.stderr


def test_random_weights_command(tmp_path):
    proc = subprocess.run(
        [sys.executable, "-m", "railgun_b200", "random-weights", "--config",
         str(helpers.model_dir("B") / "config.json"), "--seed", "2", "--out", str(tmp_path / "m"), "--std", "0.1"],
        capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    a = P.read_safetensors(tmp_path / "m" / "model.safetensors")
    b = P.read_safetensors(helpers.model_dir("B") / "model.safetensors")
    assert set(a) == set(b) and all(np.array_equal(a[k], b[k]) for k in a)
