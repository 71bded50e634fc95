"""The decode-attention entry point for callers that cannot allocate.

Some callers of this library may not call cudaMalloc: a host program that has
given all device memory to its own pool, or a plugin running where an
allocation could stall the device.  For them the library exports
``rg_decode_attention_static_scratch``, whose scratch is a fixed 4 MiB array
inside the library.  This test calls it through its exported C symbol, the
way such a caller would, twice in a row with different inputs, and checks it
against the ordinary entry point (``ops.decode_attention``, which allocates
its scratch); then that it refuses work that would not fit the array.

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
