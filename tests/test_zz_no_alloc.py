"""The decode-attention entry point for callers that cannot allocate.

Some callers of this library may not call cudaMalloc: a host program that has
given all device memory to its own pool, or a plugin running where an
allocation could stall the device.  For them the library exports
``rg_decode_attention_static_scratch``, whose scratch is a fixed 4 MiB array
inside the library.  This test calls it through its exported C symbol, the
way such a caller would, twice in a row with different inputs, and checks it
against the ordinary entry point (``ops.decode_attention``, which allocates
its scratch) and against a 64-bit restatement of the attention formula; then
a sequence of calls whose counters land where an earlier, larger call left
partial results; then that it refuses work that would not fit the array.

The file's name makes pytest collect it last, so a run that stops at the first
failure has already run every other test.
"""
import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, n_req, ctx, nh, nkv, d, page):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // page) for c in ctx]
    n_pages = sum(blocks) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.zeros(n_req, max(blocks), dtype=torch.int32)
    k = 0
    for r, b in enumerate(blocks):
        bt[r, :b] = torch.tensor(perm[k:k + b], dtype=torch.int32)
        k += b
    kv = torch.randn(n_pages, 2, nkv, page, d, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(n_req, nh * d, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([c - 1 for c in ctx], dtype=torch.int32, device=DEV)
    req = torch.arange(n_req, dtype=torch.int32, device=DEV)
    return q, kv, bt.to(DEV), req, pos


def _call_static(lib, q, out, kv, bt, req, pos, nh, nkv, d, page, splits):
    fn = lib.rg_decode_attention_static_scratch
    fn.restype = c_int
    msg = ctypes.create_string_buffer(512)
    code = fn(c_void_p(q.data_ptr()), c_int(q.shape[1]), c_void_p(out.data_ptr()), c_void_p(kv.data_ptr()),
              c_void_p(bt.data_ptr()), c_int(bt.shape[1]), c_void_p(0), c_int(q.shape[0]), c_void_p(req.data_ptr()),
              c_void_p(pos.data_ptr()), c_int(nh), c_int(nkv), c_int(d), c_int(page), c_int(0),
              c_float(d ** -0.5), c_int(splits), c_void_p(torch.cuda.current_stream().cuda_stream),
              msg, c_int(512))
    return code, msg.value.decode()


def test_static_scratch_entry_point_matches_the_allocating_one():
    from railgun_b200 import native, ops
    lib = native.load("attention_mma")
    # two calls in a row: different sizes, head counts and split counts, so stale scratch would show
    for seed, (n_req, ctx, nh, nkv, d, page, splits) in enumerate([
            (5, [700, 33, 1, 257, 128], 8, 2, 64, 16, 6),
            (3, [90, 1500, 64], 12, 4, 128, 32, 3)]):
        q, kv, bt, req, pos = _case(seed, n_req, ctx, nh, nkv, d, page)
        want = torch.empty(n_req, nh * d, dtype=torch.bfloat16, device=DEV)
        ops.decode_attention(q, nh * d, want, kv, bt, None, n_req, req, pos, nh, nkv, d, 0, d ** -0.5, splits)
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        code, msg = _call_static(lib, q, got, kv, bt, req, pos, nh, nkv, d, page, splits)
        torch.cuda.synchronize()
        assert code == 0, msg
        assert torch.cuda.memory_allocated() == before
        err = (got.double() - want.double()).abs().max() / want.double().abs().max()
        assert err < 1e-2, f"call {seed}: relative error {err:.3e}"      # the tolerance of the kernel tests
        ref = _reference(q, kv, bt, pos, nh, nkv, d, page)
        err = (got.double().cpu() - ref).abs().max() / ref.abs().max()
        assert err < 1e-2, f"call {seed}: relative error {err:.3e} against the 64-bit formula"


def _reference(q, kv, bt, pos, nh, nkv, d, page):
    """softmax(q . k / sqrt(d)) v over each request's keys, in 64-bit, from the paged cache."""
    q, kv = q.double().cpu(), kv.double().cpu()
    out = torch.zeros(q.shape[0], nh, d, dtype=torch.float64)
    for r in range(q.shape[0]):
        idx = torch.arange(int(pos[r]) + 1)
        pages = bt[r].cpu().long()[idx // page]
        K, V = kv[pages, 0, :, idx % page, :], kv[pages, 1, :, idx % page, :]
        for h in range(nh):
            kh = h // (nh // nkv)
            p = torch.softmax((K[:, kh, :] @ q[r, h * d:(h + 1) * d]) * d ** -0.5, dim=0)
            out[r, h] = p @ V[:, kh, :]
    return out.reshape(q.shape[0], nh * d)


def test_static_scratch_counters_do_not_inherit_an_earlier_calls_results():
    """A large call fills the array with partial results; the calls after it are small, need the same number of
    partial results as one another but different numbers of counters (8 key/value heads, then 32; one token with
    4 splits, then two tokens with 2 splits), so their counters lie where the large call wrote.  Every output row
    must be written (they start as NaN) and match the 64-bit formula."""
    from railgun_b200 import native
    lib = native.load("attention_mma")
    cases = [(40, [300] * 40, 32, 8, 64, 16, 7),                  # large: 40 x 32 x 7 x 66 floats = 2.4 MB
             (2, [500, 90], 32, 8, 64, 16, 2),
             (2, [260, 41], 32, 32, 64, 16, 2),                   # as many partial results, four times the counters
             (1, [700], 32, 8, 64, 16, 4),
             (2, [130, 700], 32, 8, 64, 16, 2)]
    for seed, (n_req, ctx, nh, nkv, d, page, splits) in enumerate(cases):
        q, kv, bt, req, pos = _case(40 + seed, n_req, ctx, nh, nkv, d, page)
        got = torch.full((n_req, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        code, msg = _call_static(lib, q, got, kv, bt, req, pos, nh, nkv, d, page, splits)
        torch.cuda.synchronize()
        assert code == 0, msg
        assert not torch.isnan(got).any(), f"call {seed}: rows were left unwritten"
        if n_req <= 2:
            want = _reference(q, kv, bt, pos, nh, nkv, d, page)
            err = (got.double().cpu() - want).abs().max() / want.abs().max()
            assert err < 1e-2, f"call {seed}: relative error {err:.3e}"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from railgun_b200 import native
    lib = native.load("attention_mma")
    n_req, nh, nkv, d, page = 64, 32, 8, 128, 16
    q, kv, bt, req, pos = _case(9, n_req, [40] * n_req, nh, nkv, d, page)
    out = torch.zeros(n_req, nh * d, dtype=torch.bfloat16, device=DEV)
    code, msg = _call_static(lib, q, out, kv, bt, req, pos, nh, nkv, d, page, 8)   # 64*32*8*130*4 = 8.5 MB
    torch.cuda.synchronize()
    assert code == 10002 and "fixed array holds 4194304" in msg
    assert not out.any()                                                # nothing was launched
    code, msg = _call_static(lib, q, out, kv, bt, req, pos, nh, 0, d, page, 2)     # no key/value heads: refused
    assert code == 10001 and "num_kv_heads" in msg
