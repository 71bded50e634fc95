"""Each kernel alone against a plain PyTorch reference of the same operation,
at sizes other than the engine's (widths and vocabularies that are no power of
two, head sizes in steps of 16, any number of heads and groups)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


TOL = {torch.float32: 2e-6, torch.bfloat16: 1e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 200, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, 1000, (77,), generator=g, dtype=torch.int32).to(DEV)
    out = ops.embedding(ids, table)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("H", [96, 200, 2048, 5000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(H, dtype):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(H)
    T = 13
    resid = torch.randn(T, H, generator=g).to(DEV)
    pend = torch.randn(T, H, generator=g).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(DEV)
    eps = 1e-5
    ref_sum = resid.double() + pend.double()
    ref = ref_sum / torch.sqrt((ref_sum ** 2).mean(-1, keepdim=True) + eps) * w.double()
    r = resid.clone()
    out = ops.add_rmsnorm(r, pend, w, eps, dtype)
    assert out.dtype == dtype and rel_err(out, ref) < TOL[dtype]
    assert rel_err(r, ref_sum) < 1e-7                         # the residual stream holds the 32-bit sum
    # no pending: plain norm, residual untouched
    r = resid.clone()
    out = ops.add_rmsnorm(r, None, w, eps, dtype)
    ref0 = resid.double() / torch.sqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps) * w.double()
    assert rel_err(out, ref0) < TOL[dtype] and torch.equal(r, resid)
    # selected rows only, residual untouched
    rows = torch.tensor([12, 0, 5, 5], dtype=torch.int32, device=DEV)
    r = resid.clone()
    out = ops.add_rmsnorm(r, pend, w, eps, dtype, rows=rows)
    assert out.shape == (4, H) and rel_err(out, ref[rows.long()]) < TOL[dtype] and torch.equal(r, resid)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_add_and_silu_mul(dtype):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(3)
    resid = torch.randn(9, 176, generator=g).to(DEV)
    pend = torch.randn(9, 176, generator=g).to(dtype).to(DEV)
    r = resid.clone()
    ops.residual_add(r, pend)
    assert rel_err(r, resid.double() + pend.double()) < 1e-7
    for I in (176, 1000):
        gu = (3 * torch.randn(11, 2 * I, generator=g)).to(dtype).to(DEV)
        out = ops.silu_mul(gu)
        a, b = gu[:, :I].double(), gu[:, I:].double()
        assert out.shape == (11, I) and rel_err(out, a / (1 + torch.exp(-a)) * b) < TOL[dtype]


def make_paged_case(R, ctx_lens, q_lens, nh, nkv, d, page, dtype, seed, shuffle=True, spare_pages=5):
    """Random cache contents behind shuffled block tables; the step's queries
    are the last q_lens[r] positions of each request."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // page) for c in ctx_lens]
    NP = sum(blocks) + spare_pages
    perm = torch.randperm(NP, generator=g).tolist() if shuffle else list(range(NP))
    tables, k = [], 0
    for b in blocks:
        tables.append(perm[k:k + b])
        k += b
    MB = max(blocks)
    bt = torch.zeros(R, MB, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
    kv = torch.randn(NP, 2, nkv, page, d, generator=g).to(dtype)
    positions, req = [], []
    for r in range(R):
        positions += list(range(ctx_lens[r] - q_lens[r], ctx_lens[r]))
        req += [r] * q_lens[r]
    T = len(positions)
    q = torch.randn(T, nh, d, generator=g).to(dtype)
    return dict(kv=kv, bt=bt, tables=tables, positions=positions, req=req, q=q, T=T)


def attention_reference(case, nh, nkv, d, page, window, scale):
    kv, q = case["kv"].double(), case["q"].double()
    out = torch.zeros(case["T"], nh, d, dtype=torch.float64)
    for t, (p, r) in enumerate(zip(case["positions"], case["req"])):
        lo = max(0, p - window + 1) if window else 0
        idx = torch.arange(lo, p + 1)
        pages = torch.tensor(case["tables"][r])[idx // page]
        K = kv[pages, 0, :, idx % page, :]                      # [n, nkv, d]
        V = kv[pages, 1, :, idx % page, :]
        for h in range(nh):
            kh = h // (nh // nkv)
            s = (K[:, kh, :] @ q[t, h]) * scale
            pr = torch.softmax(s, dim=0)
            out[t, h] = pr @ V[:, kh, :]
    return out.reshape(case["T"], nh * d)


ATT_CASES = [
    # nh, nkv, d, page, ctx_lens, q_lens, window
    (4, 2, 16, 16, [5, 33, 17], [5, 1, 4], 0),
    (6, 2, 48, 8, [70, 9, 130, 1], [1, 9, 7, 1], 0),
    (5, 5, 64, 16, [300, 41], [1, 41], 0),
    (8, 1, 128, 32, [257, 64, 100], [2, 1, 33], 0),
    (3, 1, 256, 16, [50, 20], [3, 20], 0),
    (4, 2, 80, 16, [200, 77, 150], [1, 30, 2], 24),
    (2, 2, 112, 4, [37], [37], 0),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case_id", range(len(ATT_CASES)))
def test_paged_attention_general(case_id, dtype):
    from railgun_b200 import ops
    nh, nkv, d, page, ctx, ql, window = ATT_CASES[case_id]
    c = make_paged_case(len(ctx), ctx, ql, nh, nkv, d, page, dtype, seed=case_id)
    scale = d ** -0.5
    ref = attention_reference(c, nh, nkv, d, page, window, scale)
    q = c["q"].reshape(c["T"], nh * d).contiguous().to(DEV)
    out = ops.paged_attention_general(
        q, nh * d, c["kv"].to(DEV), c["bt"].to(DEV), torch.tensor(c["req"], dtype=torch.int32, device=DEV),
        torch.tensor(c["positions"], dtype=torch.int32, device=DEV), nh, nkv, d, window, scale)
    assert rel_err(out, ref) < (5e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key_among_hundreds(dtype):
    """One key far back is made to dominate; losing it (a wrong page, an
    off-by-one at a page's edge) would change the output completely."""
    from railgun_b200 import ops
    nh, nkv, d, page = 4, 2, 64, 16
    ctx = [700]
    for needle in (0, 15, 16, 351, 699 - 1):
        c = make_paged_case(1, ctx, [1], nh, nkv, d, page, dtype, seed=needle)
        pg, off = c["tables"][0][needle // page], needle % page
        c["kv"][pg, 0] *= 0.05                                  # quieten that page's other keys
        c["kv"][pg, 0, :, off, :] = (c["q"][0, ::2, :] * 4).to(dtype)   # key = 4 x the query of heads 0 and 2
        ref = attention_reference(c, nh, nkv, d, page, 0, d ** -0.5)
        vneedle = c["kv"][pg, 1, :, off, :].double()
        assert (ref.reshape(nh, d)[0] - vneedle[0]).abs().max() < 0.05       # the needle's value comes out
        out = ops.paged_attention_general(
            c["q"].reshape(1, nh * d).to(DEV), nh * d, c["kv"].to(DEV), c["bt"].to(DEV),
            torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([699], dtype=torch.int32, device=DEV),
            nh, nkv, d, 0, d ** -0.5)
        assert rel_err(out, ref) < (5e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,page", [(5, 1, 48, 8), (4, 2, 16, 16), (3, 3, 128, 32)])
def test_rope_and_cache_write(nh, nkv, d, page, dtype):
    from railgun_b200 import ops
    from railgun_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(d)
    T, NP, max_pos = 21, 9, 300
    scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    table = rope_table(d, 500000.0, scaling, max_pos)
    inv = P.rope_inv_freq(d, 500000.0, dict(scaling, rope_type="llama3"))
    ang = np.arange(max_pos)[:, None] * inv[None, :]
    assert np.abs(table[:, :d // 2].double().numpy() - np.cos(ang)).max() < 1e-6      # the table is the plain angles
    assert np.abs(table[:, d // 2:].double().numpy() - np.sin(ang)).max() < 1e-6
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(dtype)
    positions = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(NP * page, generator=g)[:T].to(torch.int32)
    slots[3] = -1                                               # a token whose keys are not stored
    kv = torch.zeros(NP, 2, nkv, page, d, dtype=dtype)
    x = qkv.double().numpy().reshape(T, nh + 2 * nkv, d)
    ref_q = P.rope(x[:, :nh], positions.numpy(), inv)
    ref_k = P.rope(x[:, nh:nh + nkv], positions.numpy(), inv)
    ref_v = x[:, nh + nkv:]
    qkv_d, kv_d = qkv.to(DEV), kv.to(DEV)
    ops.rope_cache_write(qkv_d, table.to(DEV), positions.to(DEV), slots.to(DEV), kv_d, nh, nkv, d, page)
    got = qkv_d.cpu().double().numpy().reshape(T, nh + 2 * nkv, d)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert np.abs(got[:, :nh] - ref_q).max() / np.abs(ref_q).max() < tol
    assert np.array_equal(got[:, nh + nkv:], ref_v)             # v untouched
    kvc = kv_d.cpu().double().numpy()
    written = np.zeros((NP, page), dtype=bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        pg, off = divmod(s, page)
        written[pg, off] = True
        assert np.abs(kvc[pg, 0, :, off] - ref_k[t]).max() / np.abs(ref_k).max() < tol
        assert np.array_equal(kvc[pg, 1, :, off], ref_v[t])
    untouched = np.transpose(kvc, (0, 3, 1, 2, 4))[~written]    # [page, offset] first
    assert not untouched.any()                                  # nothing else was touched
    # no table: no rotation, still written
    qkv_d2, kv_d2 = qkv.to(DEV), kv.to(DEV)
    ops.rope_cache_write(qkv_d2, None, positions.to(DEV), slots.to(DEV), kv_d2, nh, nkv, d, page)
    assert torch.equal(qkv_d2.cpu(), qkv)
    s0 = int(slots[0])
    assert torch.equal(kv_d2.cpu()[s0 // page, 0, :, s0 % page].reshape(-1), qkv[0, nh * d:(nh + nkv) * d])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,page", [(5, 1, 48, 8), (4, 2, 16, 16), (3, 3, 128, 32)])
def test_rope_in_the_paired_row_order(nh, nkv, d, page, dtype):
    """The same rotation when every head's features are stored in the order that puts 8 whole pairs into every 16
    features: the results are the standard ones, reordered."""
    from railgun_b200 import ops
    from railgun_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(d + nh)
    T, NP, max_pos = 13, 5, 200
    table = rope_table(d, 10000.0, None, max_pos).to(DEV)
    order = ops.rope_pair_order(d)
    assert sorted(order.tolist()) == list(range(d))
    pairs = order.view(d // 16, 2, 8)                           # every 16 stored features: 8 firsts, then their partners
    assert torch.equal(pairs[:, 1], pairs[:, 0] + d // 2)
    qkv = torch.randn(T, nh + 2 * nkv, d, generator=g).to(dtype)
    stored = qkv.clone()
    stored[:, :nh + nkv] = qkv[:, :nh + nkv][:, :, order]       # q and k heads reordered, v as it is
    positions = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32).to(DEV)
    slots = torch.randperm(NP * page, generator=g)[:T].to(torch.int32).to(DEV)
    a, kv_a = qkv.reshape(T, -1).to(DEV), torch.zeros(NP, 2, nkv, page, d, dtype=dtype, device=DEV)
    b, kv_b = stored.reshape(T, -1).to(DEV), torch.zeros(NP, 2, nkv, page, d, dtype=dtype, device=DEV)
    ops.rope_cache_write(a, table, positions, slots, kv_a, nh, nkv, d, page)
    ops.rope_cache_write(b, table, positions, slots, kv_b, nh, nkv, d, page, paired8=True)
    a, b = a.view(T, nh + 2 * nkv, d).cpu(), b.view(T, nh + 2 * nkv, d).cpu()
    assert torch.equal(b[:, :nh + nkv], a[:, :nh + nkv][:, :, order]) and torch.equal(b[:, nh + nkv:], a[:, nh + nkv:])
    assert torch.equal(kv_b[:, 0].cpu(), kv_a[:, 0].cpu()[..., order]) and torch.equal(kv_b[:, 1], kv_a[:, 1])
    with pytest.raises(ops.KernelError):
        ops.rope_pair_order(24)


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("nh,nkv,d,K,page", [(4, 2, 64, 256, 16), (32, 8, 64, 2048, 16), (6, 3, 48, 136, 8), (40, 8, 128, 1024, 32)])
def test_projection_with_rotation_and_cache_write_in_its_kernel(M, nh, nkv, d, K, page):
    """q|k|v projection of a few single tokens, rotated and written to the cache by the product's own kernel,
    against the product followed by the rope kernel, and against 64-bit arithmetic; from plain rows and from rows
    whose norm the product finishes."""
    from railgun_b200 import ops
    from railgun_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(M + nh + d + K)
    N, NP, max_pos = (nh + 2 * nkv) * d, 7, 300
    table = rope_table(d, 500000.0, None, max_pos).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    positions = torch.randint(0, max_pos, (M,), generator=g, dtype=torch.int32).to(DEV)
    slots = torch.randperm(NP * page, generator=g)[:M].to(torch.int32)
    if M > 2:
        slots[1] = -1                                           # a token whose keys are not stored
    slots = slots.to(DEV)

    def check(x):
        kv_f = torch.zeros(NP, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
        kv_u = torch.zeros_like(kv_f)
        fused = ops.skinny_gemm_rope_cache(x, w, table, positions, slots, kv_f, nh, nkv, d)
        plain = ops.linear(x, w)                                # a NormedRows goes through the norm-finishing product
        exact = plain.double().clone()
        ops.rope_cache_write(plain, table, positions, slots, kv_u, nh, nkv, d, page, paired8=True)
        # the unfused route rounds the projection to bfloat16 before it rotates: equal within that rounding
        assert rel_err(fused[:, :nh * d], plain[:, :nh * d].double()) < 1e-2
        assert rel_err(kv_f, kv_u.double()) < 1e-2
        used = kv_u != 0
        assert torch.equal(kv_f != 0, used)                     # the same places written, nothing else
        # against the rotation in 64-bit of the unrounded... (here: of the rounded projection; one rounding apart)
        q = exact[:, :nh * d].view(M, nh, d)
        i = ops.rope_pair_order(d).to(DEV)
        inv_order = torch.argsort(i)
        std = q[:, :, inv_order]                                # back to the model's feature order
        ang = table[positions.long()].double()
        c, sn = ang[:, None, :d // 2], ang[:, None, d // 2:]
        rot = torch.cat([std[..., :d // 2] * c - std[..., d // 2:] * sn, std[..., d // 2:] * c + std[..., :d // 2] * sn], -1)
        assert rel_err(fused[:, :nh * d].view(M, nh, d)[:, :, inv_order], rot) < 1e-2

    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    check(x)
    # rows whose norm is finished inside the product
    wp = (torch.randn(K, 64, generator=g) / 8).to(torch.bfloat16).to(DEV)
    resid = torch.randn(M, K, generator=g).to(DEV)
    rows = ops.skinny_gemm_residual(torch.randn(M, 64, generator=g).to(torch.bfloat16).to(DEV), wp, resid,
                                    (torch.rand(K, generator=g) + 0.5).to(DEV), 1e-5)
    check(rows)
    # without slots nothing is written
    kv = torch.zeros(NP, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    ops.skinny_gemm_rope_cache(x, w, table, positions, None, kv, nh, nkv, d)
    assert not kv.any()
    assert not ops.skinny_rope_ok(torch.zeros(ops.SKINNY_AUTO_ROWS + 1, K, dtype=torch.bfloat16, device=DEV), w, d)
    assert not ops.skinny_rope_ok(x, w, 24)


@pytest.mark.parametrize("V", [1000, 128256])
def test_argmax_with_ties(V):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(5, V, generator=g)
    logits[1, 700] = logits[1, 33] = 9.0                        # a tie: the lowest index wins
    logits[2, V - 1] = 11.0
    logits[3, 0] = 12.0
    out = ops.argmax(logits.to(DEV)).cpu()
    ref = torch.tensor([int(np.argmax(r.numpy())) for r in logits], dtype=torch.int32)
    assert torch.equal(out, ref) and out[1] == 33


def _plain_interval(logits, temperature, top_k, top_p, tok):
    p = P.filtered_probs(logits, temperature, top_k, top_p)
    c = np.cumsum(p)
    return (c[tok] - p[tok]) / c[-1], c[tok] / c[-1], p


@pytest.mark.parametrize("V,scale", [(500, 2.5), (20001, 2.5), (128256, 2.5), (128256, 9.0)])
def test_temperature_top_k_top_p_sampling(V, scale):
    """Vocabularies that one block takes and that a cluster of blocks shares (one of them no multiple of
    four, so the last block's part is ragged); flat and peaked rows; filters that leave a handful of
    candidates (finished in shared memory) and filters that leave thousands (finished over the row)."""
    from railgun_b200 import ops
    rng = np.random.default_rng(V + int(scale))
    rows = 64
    logits = (rng.normal(size=(rows, V)) * scale).astype(np.float32)
    temperature = rng.choice([0.0, 0.5, 0.8, 1.3], size=rows).astype(np.float32)
    top_k = rng.choice([0, 1, 5, 50, 2000, V + 10], size=rows).astype(np.int32)
    top_p = rng.choice([1.0, 0.9, 0.5, 0.2], size=rows).astype(np.float32)
    seed = rng.integers(0, 2 ** 62, size=rows)
    counter = rng.integers(0, 1000, size=rows)
    dev = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)
    args = (dev(logits, torch.float32), dev(temperature, torch.float32), dev(top_k, torch.int32),
            dev(top_p, torch.float32), dev(seed, torch.int64), dev(counter, torch.int64))
    out = ops.sample(*args).cpu().numpy()
    again = ops.sample(*args).cpu().numpy()
    assert np.array_equal(out, again)                           # same seed and counter: same token
    exact = 0
    for i in range(rows):
        if temperature[i] == 0.0:
            assert out[i] == int(np.argmax(logits[i]))
            continue
        lo, hi, p = _plain_interval(logits[i], float(temperature[i]), int(top_k[i]), float(top_p[i]), int(out[i]))
        assert p[out[i]] > 0, f"row {i}: token {out[i]} is outside the kept set"
        u = P.uniform_from_counter(int(seed[i]), int(counter[i]))
        slack = 1e-4                                            # 32-bit sums over the vocabulary
        assert lo - slack <= u <= hi + slack, f"row {i}: u={u} not in [{lo}, {hi}]"
        exact += int(out[i] == P.sample(logits[i], float(temperature[i]), int(seed[i]), int(counter[i]),
                                        int(top_k[i]), float(top_p[i])))
    assert exact >= 0.9 * (temperature > 0).sum()
    # a batch of one gives the same token as the row in the big batch
    one = ops.sample(*(a[7:8].contiguous() for a in args)).cpu().numpy()
    assert one[0] == out[7]


def test_sampling_with_ties_at_the_thresholds():
    """Rows made so that the filters' thresholds fall on ties: top-k keeps every logit equal to the k-th
    largest, top-p every probability equal to its threshold; one row is constant (everything ties: the
    kept set is the whole vocabulary however small k is)."""
    from railgun_b200 import ops
    V, n = 40000, 400
    rng = np.random.default_rng(3)
    base = (rng.normal(size=V) * 0.5).astype(np.float32)
    tied = base.copy()
    top = rng.choice(V, size=30, replace=False)
    tied[top[:10]] = 6.0
    tied[top[10:]] = 5.0                                         # 20 logits tie for places 11..30
    const = np.full(V, 1.25, dtype=np.float32)
    cases = [(tied, 15, 1.0, set(top.tolist())),                 # k = 15 falls inside the tie: all 30 kept
             (tied, 10, 1.0, set(top[:10].tolist())),
             (tied, 0, 0.6, None), (const, 7, 1.0, None), (const, 0, 0.3, None)]
    for row, k, p, allowed in cases:
        logits = torch.tensor(np.tile(row, (n, 1)), device=DEV)
        out = ops.sample(logits, torch.full((n,), 1.0, device=DEV), torch.full((n,), k, dtype=torch.int32, device=DEV),
                         torch.full((n,), p, device=DEV), torch.full((n,), 11, dtype=torch.int64, device=DEV),
                         torch.arange(n, dtype=torch.int64, device=DEV)).cpu().numpy()
        probs = P.filtered_probs(row, 1.0, k, p)
        assert (probs[out] > 0).all(), (k, p)
        if allowed is not None:
            assert set(out.tolist()) <= allowed and len(set(out.tolist())) > len(allowed) // 2
        if row is const:
            # every token is as likely as any other: the draws spread over the whole vocabulary
            assert out.min() < V // 10 and out.max() > V - V // 10
        for i in range(0, n, 37):
            lo, hi, _ = _plain_interval(row, 1.0, k, p, int(out[i]))
            u = P.uniform_from_counter(11, i)
            assert lo - 1e-4 <= u <= hi + 1e-4


def test_sampling_follows_the_distribution():
    from railgun_b200 import ops
    rng = np.random.default_rng(9)
    V, n = 40, 4000
    row = (rng.normal(size=V) * 2).astype(np.float32)
    logits = torch.tensor(np.tile(row, (n, 1)), device=DEV)
    t = torch.full((n,), 0.9, device=DEV)
    out = ops.sample(logits, t, None, None, torch.full((n,), 5, dtype=torch.int64, device=DEV),
                     torch.arange(n, dtype=torch.int64, device=DEV)).cpu().numpy()
    freq = np.bincount(out, minlength=V) / n
    assert np.abs(freq - P.filtered_probs(row, 0.9)).max() < 0.03


def test_kernels_refuse_what_they_cannot_do():
    from railgun_b200 import ops
    with pytest.raises(ops.KernelError):
        ops.embedding(torch.zeros(3, dtype=torch.int32), torch.zeros(4, 4))          # CPU tensors: no CPU path
    with pytest.raises(ops.KernelError):
        ops.silu_mul(torch.zeros(3, 4, dtype=torch.float16, device=DEV))             # unsupported dtype
    with pytest.raises(ops.KernelError):
        ops.add_rmsnorm(torch.zeros(2, 8, device=DEV), None, torch.ones(7, device=DEV), 1e-5, torch.float32)
    kv = torch.zeros(2, 2, 1, 16, 272, device=DEV)
    with pytest.raises(ops.KernelError):                                               # head size above the limit
        ops.paged_attention_general(torch.zeros(1, 272, device=DEV), 272, kv, torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV), 1, 1, 272, 0, 1.0)


# ---- the tensor-core attention kernels (bfloat16) -------------------------------------------------------

MMA_CASES = ATT_CASES + [
    # nh, nkv, d, page, ctx_lens, q_lens, window
    (32, 8, 64, 16, [1024, 130, 64, 65], [1, 130, 64, 3], 0),       # the 1B model's shape; a prompt over three tiles
    (40, 2, 32, 16, [150, 90], [150, 1], 0),                        # 20 heads per kv head: two head tiles
    (6, 3, 96, 16, [500], [200], 64),                               # window shorter than a key tile span
    (4, 4, 16, 1, [70, 3], [70, 3], 0),                             # a page per token
    (2, 1, 160, 16, [333, 47], [77, 47], 100),
    (16, 8, 128, 64, [2000, 1], [1, 1], 0),
]


def _tiles_of(q_lens):
    tiles, off = [], 0
    for r, n in enumerate(q_lens):
        for k in range(0, n, 64):
            tiles.append((off + k, min(64, n - k), r))
        off += n
    return torch.tensor(tiles, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("case_id", range(len(MMA_CASES)))
def test_prefill_attention_mma(case_id):
    from railgun_b200 import ops
    nh, nkv, d, page, ctx, ql, window = MMA_CASES[case_id]
    c = make_paged_case(len(ctx), ctx, ql, nh, nkv, d, page, torch.bfloat16, seed=100 + case_id)
    scale = d ** -0.5
    ref = attention_reference(c, nh, nkv, d, page, window, scale)
    # q sits inside a wider buffer, as in the fused qkv projection
    wide = torch.zeros(c["T"], (nh + 2 * nkv) * d, dtype=torch.bfloat16)
    wide[:, :nh * d] = c["q"].reshape(c["T"], nh * d)
    out = torch.full((c["T"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.prefill_attention(wide.to(DEV), wide.shape[1], out, c["kv"].to(DEV), c["bt"].to(DEV), _tiles_of(ql),
                          torch.tensor(c["positions"], dtype=torch.int32, device=DEV), nh, nkv, d, window, scale)
    assert rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("case_id", range(len(MMA_CASES)))
def test_decode_attention_mma(case_id, splits):
    """Every token row treated as a single token attending up to its own position."""
    from railgun_b200 import ops
    nh, nkv, d, page, ctx, ql, window = MMA_CASES[case_id]
    c = make_paged_case(len(ctx), ctx, ql, nh, nkv, d, page, torch.bfloat16, seed=200 + case_id)
    scale = d ** -0.5
    ref = attention_reference(c, nh, nkv, d, page, window, scale)
    T = c["T"]
    q = c["q"].reshape(T, nh * d).contiguous().to(DEV)
    out = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    req = torch.tensor(c["req"], dtype=torch.int32, device=DEV)
    pos = torch.tensor(c["positions"], dtype=torch.int32, device=DEV)
    ops.decode_attention(q, nh * d, out, c["kv"].to(DEV), c["bt"].to(DEV), None, T, req, pos, nh, nkv, d, window,
                         scale, splits, fused_reduce=True)
    assert rel_err(out, ref) < 1e-2
    # the reduction as a second kernel gives the same numbers as the one fused into the last block
    two = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.decode_attention(q, nh * d, two, c["kv"].to(DEV), c["bt"].to(DEV), None, T, req, pos, nh, nkv, d, window,
                         scale, splits, fused_reduce=False)
    assert torch.equal(two, out)
    # the splits as one cluster, added up through distributed shared memory: the same numbers again
    if 2 <= splits <= 8:
        clu = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.decode_attention(q, nh * d, clu, c["kv"].to(DEV), c["bt"].to(DEV), None, T, req, pos, nh, nkv, d, window,
                             scale, splits, cluster=True)
        assert torch.equal(clu, out)
    # and again: the counters were left at zero
    again = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.decode_attention(q, nh * d, again, c["kv"].to(DEV), c["bt"].to(DEV), None, T, req, pos, nh, nkv, d, window,
                         scale, splits, fused_reduce=True)
    assert torch.equal(again, out)
    # a subset of rows, in another order, through the row list: the other rows stay untouched
    if T >= 3:
        rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
        out2 = torch.full((T, nh * d), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.decode_attention(q, nh * d, out2, c["kv"].to(DEV), c["bt"].to(DEV), rows, 3, req, pos, nh, nkv, d,
                             window, scale, splits)
        sel = rows.long().cpu()
        assert rel_err(out2[sel], ref[sel]) < 1e-2
        rest = torch.ones(T, dtype=torch.bool)
        rest[sel] = False
        assert (out2.cpu()[rest] == 7.0).all()


@pytest.mark.parametrize("kernel", ["prefill", "decode"])
def test_mma_attention_finds_a_far_key(kernel):
    from railgun_b200 import ops
    nh, nkv, d, page = 4, 2, 64, 16
    for needle in (0, 15, 16, 63, 64, 351, 698):
        c = make_paged_case(1, [700], [1], nh, nkv, d, page, torch.bfloat16, seed=needle)
        pg, off = c["tables"][0][needle // page], needle % page
        c["kv"][pg, 0] *= 0.05
        c["kv"][pg, 0, :, off, :] = (c["q"][0, ::2, :] * 4).to(torch.bfloat16)
        ref = attention_reference(c, nh, nkv, d, page, 0, d ** -0.5)
        q = c["q"].reshape(1, nh * d).to(DEV)
        out = torch.zeros(1, nh * d, dtype=torch.bfloat16, device=DEV)
        pos = torch.tensor([699], dtype=torch.int32, device=DEV)
        if kernel == "prefill":
            ops.prefill_attention(q, nh * d, out, c["kv"].to(DEV), c["bt"].to(DEV),
                                  torch.tensor([[0, 1, 0]], dtype=torch.int32, device=DEV), pos, nh, nkv, d, 0, d ** -0.5)
        else:
            ops.decode_attention(q, nh * d, out, c["kv"].to(DEV), c["bt"].to(DEV), None, 1,
                                 torch.zeros(1, dtype=torch.int32, device=DEV), pos, nh, nkv, d, 0, d ** -0.5, 5)
        assert rel_err(out, ref) < 1e-2


def test_mma_attention_refuses_other_head_sizes_and_dtypes():
    from railgun_b200 import ops
    kv = torch.zeros(2, 2, 1, 16, 24, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError):
        ops.decode_attention(torch.zeros(1, 24, dtype=torch.bfloat16, device=DEV), 24,
                             torch.zeros(1, 24, dtype=torch.bfloat16, device=DEV), kv, z.view(1, 1), None, 1, z, z,
                             1, 1, 24, 0, 1.0, 1)
    kv32 = torch.zeros(2, 2, 1, 16, 32, device=DEV)
    with pytest.raises(ops.KernelError):
        ops.prefill_attention(torch.zeros(1, 32, device=DEV), 32, torch.zeros(1, 32, device=DEV), kv32, z.view(1, 1),
                              torch.tensor([[0, 1, 0]], dtype=torch.int32, device=DEV), z, 1, 1, 32, 0, 1.0)


# ---- the weight-streaming decode product ---------------------------------------------------------------

@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 29, 64])
@pytest.mark.parametrize("N,K", [(48, 64), (500, 96), (2048, 2048), (1000, 176), (3072, 8192), (250, 4104)])
def test_skinny_gemm(M, N, K):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w.double().T
    out = ops.skinny_gemm(x, w)
    assert out.dtype == torch.bfloat16 and rel_err(out, ref) < 1e-2
    out32 = ops.skinny_gemm(x, w, out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and rel_err(out32, ref) < 2e-5      # exact products, 32-bit sums
    # a row's result does not depend on the batch around it
    alone = ops.skinny_gemm(x[M - 1:].contiguous(), w, out_dtype=torch.float32)
    assert torch.equal(alone[0], out32[M - 1])
    # x as a strided view (rows further apart than their length)
    wide = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x
    assert torch.equal(ops.skinny_gemm(wide[:, :K], w, out_dtype=torch.float32), out32)


@pytest.mark.parametrize("M", [1, 8, 40])
@pytest.mark.parametrize("I,K", [(176, 64), (256, 96), (8192, 2048)])
def test_skinny_gemm_silu_mul_and_interleaved_storage(M, I, K):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(I + K + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    a, b = x.double() @ gate.double().T, x.double() @ up.double().T
    ref = a / (1 + torch.exp(-a)) * b
    w = ops.interleave_gate_up(gate, up)
    assert torch.equal(w[:8], gate[:8]) and torch.equal(w[8:16], up[:8]) and torch.equal(w[16:24], gate[8:16])
    fused = ops.skinny_gemm(x, w, silu_mul=True)
    assert fused.shape == (M, I) and rel_err(fused, ref) < 1e-2
    # the unfused route over the same storage (what longer batches take)
    unfused = ops.silu_mul(torch.mm(x, w.t()), interleaved=True)
    assert rel_err(unfused, ref) < 2e-2


def test_skinny_gemm_refusals():
    from railgun_b200 import ops
    w = torch.zeros(32, 20, dtype=torch.bfloat16, device=DEV)
    assert not ops.skinny_gemm_ok(torch.zeros(2, 20, dtype=torch.bfloat16, device=DEV), w)      # K % 8
    assert not ops.skinny_gemm_ok(torch.zeros(65, 24, dtype=torch.bfloat16, device=DEV), w)     # too many rows
    assert not ops.skinny_gemm_ok(torch.zeros(2, 24, device=DEV), w)                            # 32-bit
    with pytest.raises(ops.KernelError):
        ops.skinny_gemm(torch.zeros(2, 20, dtype=torch.bfloat16, device=DEV), w)
    # linear() falls through to the library product for those
    y = ops.linear(torch.ones(2, 20, dtype=torch.bfloat16, device=DEV), torch.ones(32, 20, dtype=torch.bfloat16, device=DEV))
    assert y.shape == (2, 32) and float(y[0, 0]) == 20.0


# ---- the decode product with the residual addition and the norm folded in --------------------------------

@pytest.mark.parametrize("M", [1, 3, 8, 13, 16])
@pytest.mark.parametrize("H,K", [(48, 64), (200, 136), (1000, 72), (2048, 2048), (2048, 8192), (3080, 520)])
def test_skinny_gemm_residual_then_scaled(M, H, K):
    """resid += x W^T in the product's kernel, then the next product finishes the RMSNorm of the new rows:
    against 64-bit references and against the stand-alone kernels."""
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M * 7 + H + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    resid0 = (torch.randn(M, H, generator=g) * 3).to(DEV)
    nw = (torch.rand(H, generator=g) + 0.5).to(DEV)
    eps = 1e-3
    resid = resid0.clone()
    rows = ops.skinny_gemm_residual(x, w, resid, nw, eps)
    ref_resid = resid0.double() + x.double() @ w.double().T
    assert rel_err(resid, ref_resid) < 2e-6                                    # 32-bit sums added to a 32-bit residual
    # the stand-alone route: bf16 product added inside the norm kernel (one more rounding)
    resid_b = resid0.clone()
    ops.add_rmsnorm(resid_b, ops.skinny_gemm(x, w), nw, eps, torch.bfloat16)
    assert rel_err(resid_b, ref_resid) < 5e-3
    assert torch.equal(rows.scaled, (resid * nw).to(torch.bfloat16))           # one rounding, of the 32-bit product
    ss = rows.partials[:rows.blocks, :M].double().sum(0)
    assert rel_err(ss, (resid.double() ** 2).sum(1)) < 1e-6
    assert float(rows.partials[:rows.blocks, M:].abs().max()) == 0.0 if rows.partials.shape[1] > M else True
    # a row's result does not depend on the batch around it
    alone = resid0[M - 1:].clone()
    ops.skinny_gemm_residual(x[M - 1:].contiguous(), w, alone, nw, eps)
    assert torch.equal(alone[0], resid[M - 1])
    # the consumer
    normed = ref_resid * torch.rsqrt((ref_resid ** 2).mean(1, keepdim=True) + eps) * nw.double()
    for N2, silu in ((136, False), (1008, True), (3072, False)):
        w2 = (torch.randn(N2, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(DEV)
        assert ops.skinny_scaled_ok(rows, w2) == (M <= ops.SKINNY_AUTO_ROWS)
        if M > ops.SKINNY_AUTO_ROWS:
            y = ops.linear(rows, w2)                                           # falls back to norm kernel + product
            assert rel_err(y, normed @ w2.double().T) < 1e-2
            continue
        y = ops.skinny_gemm_scaled(rows, w2, silu_mul=silu)
        z = normed @ w2.double().T
        if silu:
            z = z.view(M, N2 // 16, 2, 8)
            z = (z[:, :, 0] / (1 + torch.exp(-z[:, :, 0])) * z[:, :, 1]).reshape(M, N2 // 2)
        assert y.dtype == torch.bfloat16 and rel_err(y, z) < 1e-2
        if not silu:
            assert torch.equal(ops.linear(rows, w2), y)                        # linear() takes the unfinished norm
    assert rel_err(rows.materialize(), normed) < 1e-2


def test_skinny_fused_refusals():
    from railgun_b200 import ops
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(48, 64, dtype=torch.bfloat16, device=DEV)
    nw = torch.ones(48, device=DEV)
    assert ops.skinny_fused_ok(x, w, torch.zeros(4, 48, device=DEV))
    assert not ops.skinny_fused_ok(x, w, torch.zeros(4, 48, dtype=torch.bfloat16, device=DEV))            # residual is 32-bit
    assert not ops.skinny_fused_ok(torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV), w,
                                   torch.zeros(17, 48, device=DEV))                                      # beyond the decode sizes
    with pytest.raises(ops.KernelError):
        ops.skinny_gemm_residual(torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV), w, torch.zeros(17, 48, device=DEV),
                                 nw, 1e-5)
    with pytest.raises(ops.KernelError):
        ops.skinny_gemm_residual(x, w, torch.zeros(4, 40, device=DEV), nw, 1e-5)                         # wrong residual width


# ---- the tcgen05 / TMA matrix product -------------------------------------------------------------------

@pytest.mark.parametrize("tile", ["128x128", "128x256", "256x128", "256x256"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 300, 200), (1, 48, 64), (333, 1000, 176), (1024, 3072, 2048),
                                   (129, 257 * 8, 8 * 37), (700, 520, 4104)])
def test_tc_gemm(M, N, K, tile):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w.double().T
    out = ops.tc_gemm(x, w, tile=tile, check=True)
    assert out.dtype == torch.bfloat16 and rel_err(out, ref) < 1e-2
    out32 = ops.tc_gemm(x, w, out_dtype=torch.float32, tile=tile, check=True)
    assert rel_err(out32, ref) < 2e-5                        # exact products, 32-bit accumulation
    # x as a view with a longer row pitch
    pitch = torch.zeros(M, K + 24, dtype=torch.bfloat16, device=DEV)
    pitch[:, :K] = x
    assert torch.equal(ops.tc_gemm(pitch[:, :K], w, out_dtype=torch.float32, tile=tile, check=True), out32)


@pytest.mark.parametrize("splits", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("M,N,K", [(64, 256, 512), (17, 300, 520), (33, 3072, 2048), (1, 48, 512), (50, 2048, 8192),
                                   (64, 1000, 8 * 67)])
def test_tc_stream_gemm(M, N, K, splits):
    """The swapped-operand streaming product: every split count against the 64-bit product, rows independent of
    the batch, a longer row pitch."""
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w.double().T
    out = ops.tc_stream_gemm(x, w, splits=splits, check=True)
    assert out.dtype == torch.bfloat16 and rel_err(out, ref) < 1e-2
    out32 = ops.tc_stream_gemm(x, w, out_dtype=torch.float32, splits=splits, check=True)
    assert rel_err(out32, ref) < 2e-5                        # exact products, 32-bit accumulation
    # a row's result does not depend on what else is in the batch
    alone = ops.tc_stream_gemm(x[M // 2:M // 2 + 1].contiguous(), w, out_dtype=torch.float32, splits=splits, check=True)
    assert torch.equal(alone[0], out32[M // 2])
    pitch = torch.zeros(M, K + 24, dtype=torch.bfloat16, device=DEV)
    pitch[:, :K] = x
    assert torch.equal(ops.tc_stream_gemm(pitch[:, :K], w, out_dtype=torch.float32, splits=splits, check=True), out32)


@pytest.mark.parametrize("splits", [0, 1, 4])
@pytest.mark.parametrize("M,I,K", [(40, 504, 136 * 4), (64, 8192, 2048)])
def test_tc_stream_gemm_silu_mul(M, I, K, splits):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M + I + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    gd, ud = x.double() @ gate.double().T, x.double() @ up.double().T
    ref = gd / (1 + torch.exp(-gd)) * ud
    out = ops.tc_stream_gemm(x, ops.interleave_gate_up(gate, up), silu_mul=True, splits=splits, check=True)
    assert out.shape == (M, I) and rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("splits", [0, 1, 4])
@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("H,K", [(200, 136), (2048, 2048), (2048, 8192), (3080, 520)])
def test_tc_stream_gemm_residual_then_scaled(M, H, K, splits):
    """The streaming product for 17 to 64 rows adds to the residual in its own kernel and prepares the next
    RMSNorm; the product after it finishes the norm: against 64-bit references."""
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M * 7 + H + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    resid0 = (torch.randn(M, H, generator=g) * 3).to(DEV)
    nw = (torch.rand(H, generator=g) + 0.5).to(DEV)
    eps = 1e-3
    resid = resid0.clone()
    if -(-K // 64) < splits:
        splits = 0                                                             # too few 64-wide boxes of K to split so far
    rows = ops.tc_stream_gemm_residual(x, w, resid, nw, eps, splits=splits)
    ops.tc_gemm_check()
    ref_resid = resid0.double() + x.double() @ w.double().T
    assert rel_err(resid, ref_resid) < 2e-5        # 32-bit accumulation over all of K in the tensor core (as test_tc_gemm)
    assert torch.equal(rows.scaled, (resid * nw).to(torch.bfloat16))           # one rounding, of the 32-bit product
    ss = rows.partials[:rows.blocks, :M].double().sum(0)
    assert rows.blocks == -(-H // 128) and rel_err(ss, (resid.double() ** 2).sum(1)) < 1e-6
    # a row's result does not depend on the batch around it
    alone = resid0[M - 1:].clone()
    ops.tc_stream_gemm_residual(x[M - 1:].contiguous(), w, alone, nw, eps, splits=splits)
    assert torch.equal(alone[0], resid[M - 1])
    # the consumers
    normed = ref_resid * torch.rsqrt((ref_resid ** 2).mean(1, keepdim=True) + eps) * nw.double()
    for N2, silu in ((136, False), (1008, True), (3072, False)):
        w2 = (torch.randn(N2, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(DEV)
        y = ops.tc_stream_gemm(rows, w2, silu_mul=silu, splits=splits if -(-H // 64) >= max(splits, 1) else 0, check=True)
        z = normed @ w2.double().T
        if silu:
            z = z.view(M, N2 // 16, 2, 8)
            z = (z[:, :, 0] / (1 + torch.exp(-z[:, :, 0])) * z[:, :, 1]).reshape(M, N2 // 2)
        assert y.dtype == torch.bfloat16 and rel_err(y, z) < 1e-2
        if not silu and ops.tc_stream_scaled_ok(rows, w2):
            assert rel_err(ops.linear(rows, w2), z) < 1e-2                     # linear() takes the unfinished norm
    assert rel_err(rows.materialize(), normed) < 1e-2


@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("nh,nkv,d,K,page", [(4, 2, 64, 256, 16), (32, 8, 64, 2048, 16), (6, 3, 48, 136, 8), (40, 8, 128, 1024, 32)])
def test_tc_stream_projection_with_rotation_and_cache_write(M, nh, nkv, d, K, page):
    """The q|k|v projection of 17 to 64 single tokens, rotated and written to the cache in the streaming product's
    epilogue, against the product followed by the rope kernel; from plain rows and from rows whose norm the
    product finishes."""
    from railgun_b200 import ops
    from railgun_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(M + nh + d + K)
    N, NP, max_pos = (nh + 2 * nkv) * d, 9, 300
    table = rope_table(d, 500000.0, None, max_pos).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    positions = torch.randint(0, max_pos, (M,), generator=g, dtype=torch.int32).to(DEV)
    slots = torch.randperm(NP * page, generator=g)[:M].to(torch.int32)
    slots[1] = -1                                               # a token whose keys are not stored
    slots = slots.to(DEV)

    def check(x):
        kv_f = torch.zeros(NP, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
        kv_u = torch.zeros_like(kv_f)
        fused = ops.tc_stream_gemm_rope_cache(x, w, table, positions, slots, kv_f, nh, nkv, d)
        ops.tc_gemm_check()
        plain = ops.tc_stream_gemm(x, w, check=True)            # the same product, then the rope kernel
        ops.rope_cache_write(plain, table, positions, slots, kv_u, nh, nkv, d, page, paired8=True)
        # the unfused route rounds the projection to bfloat16 before it rotates: equal within that rounding
        assert rel_err(fused[:, :nh * d], plain[:, :nh * d].double()) < 1e-2
        assert rel_err(kv_f, kv_u.double()) < 1e-2
        assert torch.equal(kv_f != 0, kv_u != 0)                # the same places written, nothing else

    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    check(x)
    wp = (torch.randn(K, 64, generator=g) / 8).to(torch.bfloat16).to(DEV)
    resid = torch.randn(M, K, generator=g).to(DEV)
    rows = ops.tc_stream_gemm_residual(torch.randn(M, 64, generator=g).to(torch.bfloat16).to(DEV), wp, resid,
                                       (torch.rand(K, generator=g) + 0.5).to(DEV), 1e-5)
    check(rows)
    kv = torch.zeros(NP, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    ops.tc_stream_gemm_rope_cache(x, w, table, positions, None, kv, nh, nkv, d)
    assert not kv.any()
    assert not ops.tc_stream_rope_ok(x, w, 24)


def test_tc_stream_gemm_refusals():
    from railgun_b200 import ops
    x = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.KernelError):
        ops.tc_stream_gemm(x, w)                              # more than 64 rows
    with pytest.raises(ops.KernelError):
        ops.tc_stream_gemm(x[:8], w, splits=3)                # not a power of two
    with pytest.raises(ops.KernelError):
        ops.tc_stream_gemm(x[:8], w, splits=2)                # K of one box cannot be split in two
    with pytest.raises(ops.KernelError):
        ops.tc_stream_gemm(x[:8].float(), w)


@pytest.mark.parametrize("tile", ["128x256", "256x128", "256x256"])
@pytest.mark.parametrize("M,I,K", [(100, 504, 136), (1100, 8192, 2048)])
def test_tc_gemm_silu_mul(M, I, K, tile):
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(M + I + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    a, b = x.double() @ gate.double().T, x.double() @ up.double().T
    ref = a / (1 + torch.exp(-a)) * b
    out = ops.tc_gemm(x, ops.interleave_gate_up(gate, up), silu_mul=True, tile=tile, check=True)
    assert out.shape == (M, I) and rel_err(out, ref) < 1e-2


def test_tc_gemm_refusals():
    from railgun_b200 import ops
    w = torch.zeros(32, 20, dtype=torch.bfloat16, device=DEV)
    assert not ops.tc_gemm_ok(torch.zeros(2, 20, dtype=torch.bfloat16, device=DEV), w)        # K % 8
    assert not ops.tc_gemm_ok(torch.zeros(2, 24, device=DEV), torch.zeros(32, 24, device=DEV))  # 32-bit
    with pytest.raises(ops.KernelError):
        ops.tc_gemm(torch.zeros(2, 20, dtype=torch.bfloat16, device=DEV), w)
    with pytest.raises(ops.KernelError):
        ops.tc_gemm(torch.zeros(2, 24, dtype=torch.bfloat16, device=DEV),
                    torch.zeros(32, 24, dtype=torch.bfloat16, device=DEV), tile="512x512")


# ---- the tcgen05 flash attention kernel (head size 64) ----------------------------------------------------

TC_ATT_CASES = [
    # nh, nkv, page, ctx_lens, q_lens, window
    (1, 1, 16, [128], [128], 0),
    (2, 1, 16, [70], [70], 0),
    (4, 2, 16, [300, 41], [300, 41], 0),
    (8, 2, 8, [1000, 130, 64, 65], [500, 130, 64, 3], 0),          # portions that start inside a context
    (4, 4, 32, [700], [260], 100),                                 # a window
    (5, 5, 64, [129, 257], [2, 129], 0),
    (3, 1, 128, [400], [400], 37),
    (32, 8, 16, [1500], [1500], 0),                                # the 1B model's shape
]


@pytest.mark.parametrize("case_id", range(len(TC_ATT_CASES)))
def test_prefill_attention_tcgen05(case_id):
    from railgun_b200 import ops
    nh, nkv, page, ctx, ql, window = TC_ATT_CASES[case_id]
    d = 64
    c = make_paged_case(len(ctx), ctx, ql, nh, nkv, d, page, torch.bfloat16, seed=300 + case_id)
    ref = attention_reference(c, nh, nkv, d, page, window, d ** -0.5)
    wide = torch.zeros(c["T"], (nh + 2 * nkv) * d, dtype=torch.bfloat16)
    wide[:, :nh * d] = c["q"].reshape(c["T"], nh * d)
    tiles, off = [], 0
    for r, n in enumerate(ql):
        tiles += [(off + k, min(128, n - k), r) for k in range(0, n, 128)]
        off += n
    out = torch.full((c["T"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.prefill_attention_tc(wide.to(DEV), out, c["kv"].to(DEV), c["bt"].to(DEV),
                             torch.tensor(tiles, dtype=torch.int32, device=DEV),
                             torch.tensor(c["positions"], dtype=torch.int32, device=DEV), nh, nkv, d, window, d ** -0.5)
    ops.tc_gemm_check()
    assert rel_err(out, ref) < 1e-2


def test_prefill_attention_tcgen05_finds_a_far_key():
    from railgun_b200 import ops
    nh, nkv, d, page = 4, 2, 64, 16
    for needle in (0, 15, 16, 127, 128, 351, 698):
        c = make_paged_case(1, [700], [1], nh, nkv, d, page, torch.bfloat16, seed=needle)
        pg, off = c["tables"][0][needle // page], needle % page
        c["kv"][pg, 0] *= 0.05
        c["kv"][pg, 0, :, off, :] = (c["q"][0, ::2, :] * 4).to(torch.bfloat16)
        ref = attention_reference(c, nh, nkv, d, page, 0, d ** -0.5)
        q = torch.zeros(1, (nh + 2 * nkv) * d, dtype=torch.bfloat16)
        q[:, :nh * d] = c["q"].reshape(1, nh * d)
        out = torch.zeros(1, nh * d, dtype=torch.bfloat16, device=DEV)
        ops.prefill_attention_tc(q.to(DEV), out, c["kv"].to(DEV), c["bt"].to(DEV),
                                 torch.tensor([[0, 1, 0]], dtype=torch.int32, device=DEV),
                                 torch.tensor([699], dtype=torch.int32, device=DEV), nh, nkv, d, 0, d ** -0.5)
        ops.tc_gemm_check()
        assert rel_err(out, ref) < 1e-2


def test_prefill_attention_tcgen05_rescales_when_the_maximum_jumps():
    """The kernel keeps a reference maximum and raises it (rescaling what it has accumulated) only when a tile's
    weights outgrow it.  Keys that align with some queries ever more strongly make that happen several times in
    a row's life, for some rows of a warp and not for others, in interior tiles and on the diagonal."""
    from railgun_b200 import ops
    nh, nkv, d, page = 2, 1, 64, 16
    T = 300
    c = make_paged_case(1, [T], [T], nh, nkv, d, page, torch.bfloat16, seed=77)
    q = c["q"]                                                   # [T, nh, d]
    for kp, strength, row in ((70, 1.5, 299), (130, 2.5, 299), (200, 3.5, 299), (290, 5.0, 299), (100, 4.0, 150),
                              (3, 3.0, 40), (260, 4.5, 270)):
        pg, off = c["tables"][0][kp // page], kp % page
        c["kv"][pg, 0, 0, off, :] = (q[row, 0, :] * strength).to(torch.bfloat16)
    ref = attention_reference(c, nh, nkv, d, page, 0, d ** -0.5)
    wide = torch.zeros(T, (nh + 2 * nkv) * d, dtype=torch.bfloat16)
    wide[:, :nh * d] = q.reshape(T, nh * d)
    tiles = [(k, min(128, T - k), 0) for k in range(0, T, 128)]
    out = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.prefill_attention_tc(wide.to(DEV), out, c["kv"].to(DEV), c["bt"].to(DEV),
                             torch.tensor(tiles, dtype=torch.int32, device=DEV),
                             torch.tensor(c["positions"], dtype=torch.int32, device=DEV), nh, nkv, d, 0, d ** -0.5)
    ops.tc_gemm_check()
    assert rel_err(out, ref) < 1e-2
    # the rows that the needles were made for are dominated by their needle's value
    v290 = c["kv"][c["tables"][0][290 // page], 1, 0, 290 % page].double()
    assert (out[299, :d].double().cpu() - v290).abs().max() < 0.05 * v290.abs().max() + 0.05


def test_prefill_attention_tcgen05_refuses_other_shapes():
    from railgun_b200 import ops
    q = torch.zeros(4, 3 * 128, dtype=torch.bfloat16, device=DEV)
    kv128 = torch.zeros(2, 2, 1, 16, 128, dtype=torch.bfloat16, device=DEV)
    assert not ops.prefill_attention_tc_ok(q, kv128, 128, 16)                       # head size
    kv = torch.zeros(2, 2, 1, 12, 64, dtype=torch.bfloat16, device=DEV)
    assert not ops.prefill_attention_tc_ok(q, kv, 64, 12)                           # page size
    with pytest.raises(ops.KernelError):
        ops.prefill_attention_tc(q, torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV), kv,
                                 torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                 torch.tensor([[0, 4, 0]], dtype=torch.int32, device=DEV),
                                 torch.zeros(4, dtype=torch.int32, device=DEV), 1, 1, 64, 0, 1.0)


@pytest.mark.gpu
def test_probe_sm100_reports_cycles_in_range():
    """The diagnostic that times the tcgen05 kernels' building blocks runs and gives figures of the right order:
    an exponential takes 8 cycles of a scheduler's special-function unit, a tcgen05.mma of N 256 four times one of
    N 64 at most, and a wait on a completed barrier costs more with one polling lane and a shuffle."""
    from railgun_b200 import ops
    r = ops.probe_sm100(DEV)
    assert 6.0 < r["ex2.approx.ftz.f32"] < 12.0
    assert 0.5 < r["fma.rn.f32"] < 2.5
    assert 20 < r["tcgen05.mma M128 N64 K16"] <= r["tcgen05.mma M128 N128 K16"] <= r["tcgen05.mma M128 N256 K16"] < 400
    assert r["mbarrier wait (done), every lane"] < r["mbarrier wait (done), lane 0 + shuffle"]
    assert r["softmax pass of 64 columns, 1 warp per scheduler"] < r["softmax pass of 64 columns, 2 warps per scheduler"]


@pytest.mark.gpu
def test_attention_kernels_at_long_contexts():
    """Portions of prompts and single tokens far into contexts of 40,000 and 70,001 tokens (5,000 pages a request):
    the split decode kernel with one, eight and two hundred splits, and both prefill kernels, whose portions start
    hundreds of key tiles into the context."""
    from railgun_b200 import ops
    nh, nkv, d, page, ctx, ql = 8, 2, 64, 16, [40000, 70001], [256, 130]
    c = make_paged_case(len(ctx), ctx, ql, nh, nkv, d, page, torch.bfloat16, seed=5)
    scale = d ** -0.5
    ref = attention_reference(c, nh, nkv, d, page, 0, scale)
    T = c["T"]
    q = c["q"].reshape(T, nh * d).contiguous().to(DEV)
    req = torch.tensor(c["req"], dtype=torch.int32, device=DEV)
    pos = torch.tensor(c["positions"], dtype=torch.int32, device=DEV)
    kv, bt = c["kv"].to(DEV), c["bt"].to(DEV)
    for splits in (1, 8, 200):
        out = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.decode_attention(q, nh * d, out, kv, bt, None, T, req, pos, nh, nkv, d, 0, scale, splits)
        assert rel_err(out, ref) < 1e-2, splits
    out = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.prefill_attention(q, nh * d, out, kv, bt, _tiles_of(ql), pos, nh, nkv, d, 0, scale)
    assert rel_err(out, ref) < 1e-2
    wide = torch.zeros(T, (nh + 2 * nkv) * d, dtype=torch.bfloat16, device=DEV)
    wide[:, :nh * d] = q
    tiles, off = [], 0
    for r, n in enumerate(ql):
        tiles += [(off + k, min(128, n - k), r) for k in range(0, n, 128)]
        off += n
    out = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.prefill_attention_tc(wide, out, kv, bt, torch.tensor(tiles, dtype=torch.int32, device=DEV), pos, nh, nkv, d, 0, scale)
    ops.tc_gemm_check()
    assert rel_err(out, ref) < 1e-2
