"""Python entry points of the hand-written sm_100a kernels.

Each function checks its arguments (device, dtype, contiguity, sizes), calls
the ``extern "C"`` launcher on the current CUDA stream and raises on any
error.  There is no CPU path and no library fallback: without a CUDA device,
or if a library fails to build, these raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_float, c_void_p, c_longlong

import torch

from . import native

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 or bfloat16")


def _check(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device (what torch.cuda.stream and graph capture set)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ok(code: int, what: str) -> None:
    if code == 0:
        return
    if code == 10001:
        raise KernelError(f"{what}: the kernel refuses these sizes or dtypes")
    raise KernelError(f"{what}: CUDA error {code}")


class LaunchCounter:
    """Counts launches of this package's own kernels (library matrix products
    are not counted).  A replayed CUDA graph adds the launches it captured."""

    def __init__(self):
        self.value = 0


_COUNTER = LaunchCounter()
_fn_cache: dict = {}


def launch_counter() -> LaunchCounter:
    return _COUNTER


# Programmatic dependent launch: a kernel may start (and fetch weights) while the kernel before it drains.
# RAILGUN_B200_PDL=0 switches it off.
PDL_ENABLED = os.environ.get("RAILGUN_B200_PDL", "1") != "0"
_pdl_set: set = set()


def _fn(lib_name: str, fn_name: str):
    fn = _fn_cache.get(fn_name)
    if fn is None:
        lib = native.load(lib_name)
        if lib_name not in _pdl_set:
            lib.rg_set_pdl.restype = None
            lib.rg_set_pdl(c_int(1 if PDL_ENABLED else 0))
            _pdl_set.add(lib_name)
        fn = getattr(lib, fn_name)
        fn.restype = c_int
        _fn_cache[fn_name] = fn
    _COUNTER.value += 1
    return fn


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """residual [T, H] float32 = table[ids]."""
    _check(ids, "ids", torch.int32)
    _check(table, "table")
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _ok(_fn("embedding", "rg_embedding")(_ptr(ids), _ptr(table), c_int(_dtype_code(table)), _ptr(out),
                                         c_int(T), c_int(H), c_int(V), _stream()), "embedding")
    return out


def add_rmsnorm(resid: torch.Tensor, pending, weight: torch.Tensor, eps: float, out_dtype,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """resid += pending (in place, 32-bit), then RMSNorm of resid.  With
    ``rows`` (int32 indices) only those rows are normed and resid is untouched."""
    _check(resid, "resid", torch.float32)
    _check(weight, "weight", torch.float32)
    T, H = resid.shape
    if weight.numel() != H:
        raise KernelError(f"norm weight has {weight.numel()} elements, rows have {H}")
    if pending is not None:
        _check(pending, "pending")
        if pending.shape != resid.shape:
            raise KernelError(f"pending {tuple(pending.shape)} vs residual {tuple(resid.shape)}")
    n_out = T
    if rows is not None:
        _check(rows, "rows", torch.int32)
        n_out = rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=resid.device)
    _ok(_fn("norm", "rg_add_rmsnorm")(
        _ptr(resid), _ptr(pending), c_int(_dtype_code(pending) if pending is not None else 0), _ptr(weight),
        c_float(eps), _ptr(out), c_int(_dtype_code(out)), _ptr(rows), c_int(n_out), c_int(H), _stream()),
        "add_rmsnorm")
    return out


def residual_add(resid: torch.Tensor, pending: torch.Tensor) -> None:
    _check(resid, "resid", torch.float32)
    _check(pending, "pending")
    if pending.shape != resid.shape:
        raise KernelError(f"pending {tuple(pending.shape)} vs residual {tuple(resid.shape)}")
    _ok(_fn("norm", "rg_residual_add")(_ptr(resid), _ptr(pending), c_int(_dtype_code(pending)),
                                       c_longlong(resid.numel()), _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """[T, 2I] -> [T, I]: silu(gate) * up.  Plain storage: gate is the first
    half of a row, up the second.  ``interleaved``: blocks of 8 gate columns
    followed by their 8 up columns (the storage ``interleave_gate_up`` makes)."""
    _check(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2 or (interleaved and two_i % 16):
        raise KernelError("silu_mul: last dimension must be even (a multiple of 16 when interleaved)")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    name = "rg_silu_mul_interleaved" if interleaved else "rg_silu_mul"
    _ok(_fn("activation", name)(_ptr(gate_up), _ptr(out), c_int(_dtype_code(gate_up)),
                                c_int(T), c_int(two_i // 2), _stream()), "silu_mul")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate [I, K] and up [I, K] as blocks of 8 gate rows followed by the
    8 matching up rows, so that one 16-row tensor-core tile holds a gate
    element and its up element in the same thread (I % 8 == 0)."""
    I, K = gate.shape
    if I % 8 or up.shape != gate.shape:
        raise KernelError("interleave_gate_up: both [I, K] with I a multiple of 8")
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


SKINNY_MAX_ROWS = 64           # what the kernel takes
SKINNY_AUTO_ROWS = 16          # up to here it beats the library product on B200 (measured, with the fused
                               # residual / norm / rotary variants in a decoder layer), so linear() uses it


def skinny_gemm_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Can the weight-streaming decode product take this shape?"""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.is_contiguous())


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype=None, silu_mul: bool = False) -> torch.Tensor:
    """y = x W^T for up to 64 rows of x, reading W once at memory speed.
    ``silu_mul``: W is interleaved gate|up storage and y = silu(gate) * up."""
    if not skinny_gemm_ok(x, weight):
        raise KernelError(f"skinny_gemm refuses x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)} {weight.dtype}: "
                          "bfloat16, at most 64 rows, K a multiple of 8")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"skinny_gemm: x has {K} columns, W has {weight.shape[1]}")
    out_dtype = out_dtype or torch.bfloat16
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("skinny_gemm: the SiLU-mul epilogue needs N % 16 == 0 and bfloat16 output")
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    _ok(_fn("gemm_skinny", "rg_skinny_gemm")(
        _ptr(weight), _ptr(x), c_int(x.stride(0)), _ptr(out), c_int(out.shape[1]), c_int(_dtype_code(out)),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), _stream()), "skinny_gemm")
    return out


SKINNY_FUSED_MAX_ROWS = 16     # what the fused variants (residual epilogue, norm prologue) are compiled for


class NormedRows:
    """RMSNorm of the residual rows, not finished yet: ``scaled`` holds
    bf16(residual * norm weight) and ``partials`` [>= blocks, ld] the partial
    sums of squares of the residual rows, one row per block of the product that
    last added to the residual.  A product that follows multiplies its sums by
    1 / rms (``linear`` and ``skinny_gemm_scaled`` take this in place of a
    tensor); ``materialize()`` runs the norm kernel on the residual."""

    __slots__ = ("resid", "scaled", "partials", "blocks", "weight", "eps", "dtype")

    def __init__(self, resid, scaled, partials, blocks: int, weight, eps: float, dtype):
        self.resid, self.scaled, self.partials, self.blocks = resid, scaled, partials, blocks
        self.weight, self.eps, self.dtype = weight, eps, dtype

    @property
    def shape(self):
        return self.resid.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.resid, None, self.weight, self.eps, self.dtype)


class PendingLinear:
    """A part's output x W^T, not computed yet: a norm that follows adds it to
    the residual inside the product's own kernel; ``materialize()`` runs the
    product."""

    __slots__ = ("x", "weight")

    def __init__(self, x, weight):
        self.x, self.weight = x, weight

    @property
    def shape(self):
        return (self.x.shape[0], self.weight.shape[0])

    def materialize(self) -> torch.Tensor:
        return linear(self.x, self.weight)


def skinny_fused_ok(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor) -> bool:
    """Can x W^T be added to ``resid`` inside the decode product (which then
    also prepares the next norm)?  Only where ``linear`` would use that product."""
    return (x.shape[0] <= min(SKINNY_AUTO_ROWS, SKINNY_FUSED_MAX_ROWS) and skinny_gemm_ok(x, weight)
            and resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == (x.shape[0], weight.shape[0])
            and resid.shape[1] % 8 == 0)


def skinny_gemm_residual(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor,
                         eps: float) -> NormedRows:
    """resid += x W^T (32-bit, in place), and the RMSNorm (``norm_weight``,
    ``eps``) of the new rows but for the factor 1 / rms, which the product that
    reads the result applies."""
    if not (x.shape[0] <= SKINNY_FUSED_MAX_ROWS and skinny_gemm_ok(x, weight)):
        raise KernelError(f"skinny_gemm_residual refuses x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)}")
    _check(resid, "resid", torch.float32)
    _check(norm_weight, "norm_weight", torch.float32)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or resid.shape != (M, N) or norm_weight.numel() != N:
        raise KernelError(f"skinny_gemm_residual: x {tuple(x.shape)}, W {tuple(weight.shape)}, residual "
                          f"{tuple(resid.shape)}, norm weight {norm_weight.numel()}")
    ld = 8 * ((M + 7) // 8)
    partials = torch.empty(((N + 15) // 16, ld), dtype=torch.float32, device=x.device)
    scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    blocks = c_int(0)
    _ok(_fn("gemm_skinny_fused", "rg_skinny_gemm_residual")(
        _ptr(weight), _ptr(x), c_int(x.stride(0)), _ptr(resid), c_int(resid.stride(0)), _ptr(norm_weight), _ptr(scaled),
        c_int(M), c_int(N), c_int(K), _ptr(partials), c_int(ld), ctypes.byref(blocks), _stream()),
        "skinny_gemm_residual")
    return NormedRows(resid, scaled, partials, blocks.value, norm_weight, eps, torch.bfloat16)


def skinny_scaled_ok(rows: NormedRows, weight: torch.Tensor) -> bool:
    return (rows.dtype == torch.bfloat16 and rows.shape[0] <= min(SKINNY_AUTO_ROWS, SKINNY_FUSED_MAX_ROWS)
            and skinny_gemm_ok(rows.scaled, weight) and rows.shape[1] == weight.shape[1])


def skinny_gemm_scaled(rows: NormedRows, weight: torch.Tensor, silu_mul: bool = False) -> torch.Tensor:
    """y = rmsnorm(residual rows) W^T from the unfinished norm ``rows``: the
    product over the scaled rows, its 32-bit sums multiplied by 1 / rms before
    the epilogue; ``silu_mul`` as in ``skinny_gemm``.  bfloat16 out."""
    if not skinny_scaled_ok(rows, weight):
        raise KernelError(f"skinny_gemm_scaled refuses rows {tuple(rows.shape)}, W {tuple(weight.shape)} {weight.dtype}")
    x = rows.scaled
    M, K = x.shape
    N = weight.shape[0]
    if silu_mul and N % 16:
        raise KernelError("skinny_gemm_scaled: the SiLU-mul epilogue needs N % 16 == 0")
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=torch.bfloat16, device=x.device)
    _ok(_fn("gemm_skinny_fused", "rg_skinny_gemm_scaled")(
        _ptr(weight), _ptr(x), c_int(x.stride(0)), c_float(rows.eps), _ptr(rows.partials),
        c_int(rows.partials.stride(0)), c_int(rows.blocks), _ptr(out), c_int(out.shape[1]),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), _stream()), "skinny_gemm_scaled")
    return out


def rope_pair_order(d: int) -> torch.Tensor:
    """The "paired8" order of a head's features (d % 16 == 0): storage index ->
    original feature, such that rotation pair i = (i, i + d/2) sits at storage
    indices (16 (i // 8) + i % 8, + 8): every 16 consecutive features hold 8
    whole pairs.  q . k does not notice a reordering that q and k share."""
    if d % 16:
        raise KernelError(f"the paired8 order needs a head size that is a multiple of 16, not {d}")
    s = torch.arange(d)
    blk, r = s // 16, s % 16
    return torch.where(r < 8, 8 * blk + r, d // 2 + 8 * blk + (r - 8))


def reorder_rope_rows(weight: torch.Tensor, n_heads: int, d: int) -> torch.Tensor:
    """Rows of a q or k projection [n_heads * d, K] in the paired8 order."""
    order = rope_pair_order(d).to(weight.device)
    return weight.view(n_heads, d, -1)[:, order, :].reshape(n_heads * d, -1).contiguous()


def rope_cache_write(qkv: torch.Tensor, table, positions: torch.Tensor, slots, kv_cache,
                     nh: int, nkv: int, d: int, page_size: int, err_flag=None, paired8: bool = False) -> None:
    """Rotate the q and k heads of qkv [T, (nh+2nkv)d] in place by ``table``
    [max_pos, d] (None: no rotation) and write k, v to the paged cache
    [NP, 2, nkv, page_size, d] at ``slots`` (None: no write).  ``paired8``: the
    heads' features are in ``rope_pair_order``."""
    _check(qkv, "qkv")
    _check(positions, "positions", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qkv row has {qkv.shape[1]} elements, expected {(nh + 2 * nkv) * d}")
    max_pos = 1 << 30
    if table is not None:
        _check(table, "rope table", torch.float32)
        if table.shape[1] != d:
            raise KernelError(f"rope table is for head size {table.shape[1]}, heads have {d}")
        max_pos = table.shape[0]
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", qkv.dtype)
        if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match "
                              f"[pages, 2, {nkv}, {page_size}, {d}]")
    _ok(_fn("rope_cache", "rg_rope_cache")(
        _ptr(qkv), c_int(_dtype_code(qkv)), _ptr(table), _ptr(positions), _ptr(slots),
        _ptr(kv_cache if slots is not None else None), c_int(T), c_int(nh), c_int(nkv), c_int(d),
        c_int(page_size), c_int(max_pos), _ptr(err_flag), c_int(1 if paired8 else 0), _stream()), "rope_cache_write")


def skinny_gemm_rope_cache(x, weight: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, slots, kv_cache,
                           nh: int, nkv: int, d: int, err_flag=None) -> torch.Tensor:
    """The q|k|v projection of up to 8 single tokens with the rotary encoding
    and the cache write inside the product's kernel: returns [M, (nh+2nkv)d]
    whose q heads are rotated (its k and v columns are not written); k
    (rotated) and v go to ``kv_cache`` at ``slots`` (None: no write).  ``x``:
    bfloat16 rows or a ``NormedRows``; ``weight``'s q and k rows are in
    ``rope_pair_order``."""
    rows = x if isinstance(x, NormedRows) else None
    xin = rows.scaled if rows is not None else x
    if not skinny_rope_ok(x, weight, d):
        raise KernelError(f"skinny_gemm_rope_cache refuses rows {tuple(xin.shape)}, W {tuple(weight.shape)}, head size {d}")
    M, K = xin.shape
    N = weight.shape[0]
    if weight.shape[1] != K or N != (nh + 2 * nkv) * d:
        raise KernelError(f"skinny_gemm_rope_cache: W {tuple(weight.shape)} is not [({nh} + 2 x {nkv}) x {d}, {K}]")
    _check(table, "rope table", torch.float32)
    _check(positions, "positions", torch.int32)
    if table.shape[1] != d or positions.numel() < M:
        raise KernelError("skinny_gemm_rope_cache: the table's head size or the number of positions does not match")
    page_size = 0
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", torch.bfloat16)
        page_size = kv_cache.shape[3]
        if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d) or slots.numel() < M:
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match [pages, 2, {nkv}, page, {d}]")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xin.device)
    _ok(_fn("gemm_skinny_fused", "rg_skinny_gemm_rope_cache")(
        _ptr(weight), _ptr(xin), c_int(xin.stride(0)), c_float(rows.eps if rows is not None else 0.0),
        _ptr(rows.partials if rows is not None else None), c_int(rows.partials.stride(0) if rows is not None else 0),
        c_int(rows.blocks if rows is not None else 0), _ptr(out), c_int(N), c_int(M), c_int(N), c_int(K), _ptr(table),
        _ptr(positions), _ptr(slots), _ptr(kv_cache if slots is not None else None), c_int(nh), c_int(nkv), c_int(d),
        c_int(page_size), c_int(table.shape[0]), _ptr(err_flag), _stream()), "skinny_gemm_rope_cache")
    return out


def skinny_rope_ok(x, weight: torch.Tensor, d: int) -> bool:
    """Can the q|k|v projection of these rows rotate and write the cache in its own kernel?"""
    if d % 16:
        return False
    if isinstance(x, NormedRows):
        return skinny_scaled_ok(x, weight)
    return x.shape[0] <= min(SKINNY_AUTO_ROWS, SKINNY_FUSED_MAX_ROWS) and skinny_gemm_ok(x, weight)


def paged_attention_general(q: torch.Tensor, q_stride: int, kv_cache: torch.Tensor, block_table: torch.Tensor,
                            req_of_token: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int, d: int,
                            window: int, scale: float) -> torch.Tensor:
    """The general attention kernel: out [T, nh*d].  ``q`` may be a view whose
    rows are ``q_stride`` elements apart (the q part of a fused qkv buffer)."""
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (there is no CPU path)")
    _check(kv_cache, "kv_cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    T = positions.numel()
    page_size = kv_cache.shape[3]
    if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match heads {nkv} x {d}")
    if d > 256:
        raise KernelError(f"head size {d} is above the kernels' limit of 256")
    out = torch.empty((T, nh * d), dtype=q.dtype, device=q.device)
    _ok(_fn("attention_general", "rg_paged_attention_general")(
        _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), c_int(_dtype_code(q)), _ptr(block_table),
        c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), c_int(T), c_int(nh), c_int(nkv),
        c_int(d), c_int(page_size), c_int(window or 0), c_float(scale), _stream()), "paged_attention_general")
    return out


def _check_paged(q, kv_cache, block_table, nkv, d):
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (there is no CPU path)")
    if q.dtype != torch.bfloat16:
        raise KernelError(f"the tensor-core attention kernels take bfloat16, got {q.dtype}")
    _check(kv_cache, "kv_cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    page_size = kv_cache.shape[3]
    if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match heads {nkv} x {d}")
    if d % 16 or not 16 <= d <= 256:
        raise KernelError(f"the tensor-core attention kernels take head sizes 16, 32, ..., 256; got {d}")
    return page_size


def prefill_attention(q, q_stride: int, out, kv_cache, block_table, tiles, positions, nh: int, nkv: int, d: int,
                      window: int, scale: float) -> None:
    """Flash-style attention for requests that bring several tokens: ``tiles``
    [n, 3] = (first row, rows <= 64, request index).  Writes the tiles' rows of
    ``out`` [T, nh*d]."""
    page_size = _check_paged(q, kv_cache, block_table, nkv, d)
    _check(tiles, "tiles", torch.int32)
    _check(positions, "positions", torch.int32)
    _check(out, "out", q.dtype)
    _ok(_fn("attention_mma", "rg_prefill_attention")(
        _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(tiles), c_int(tiles.shape[0]), _ptr(positions), c_int(nh), c_int(nkv), c_int(d), c_int(page_size),
        c_int(window or 0), c_float(scale), _stream()), "prefill_attention")


def decode_splits(n_tokens: int, kv_tiles: int, max_context: int) -> int:
    """How many parts each context is cut into.  Measured on B200: the split
    kernel runs best when all its thread blocks are resident at once (4 per SM,
    592 in all) and each part has at least 256 keys; more parts only add
    partial results to reduce."""
    by_residency = 592 // max(1, n_tokens * kv_tiles)
    by_length = -(-max_context // 256)
    return max(1, min(by_residency, by_length, 256))


_decode_counters: dict = {}


def decode_attention(q, q_stride: int, out, kv_cache, block_table, rows, n_tokens: int, req_of_token, positions,
                     nh: int, nkv: int, d: int, window: int, scale: float, num_splits: int,
                     scratch=None, fused_reduce=None, cluster: bool = False) -> None:
    """Split attention for single tokens: token rows ``rows`` (None: rows
    0..n_tokens-1) each attend their request's context.  Partial results go
    through scratch memory (allocated here unless given) and are reduced into
    ``out`` [T, nh*d] by the block that finishes last for each token and head
    tile (``fused_reduce``) or by a second kernel (the default: measured
    faster, the last block would reduce alone at the end of the launch); a
    single split writes the result itself.  ``cluster`` (2 to 8 splits): the
    splits of a (token, head tile) are one thread-block cluster and add their
    partial results through distributed shared memory; the fastest way for the
    kernel alone, not inside a decode step (see attention_mma.cu), so the
    engine leaves it off.  Every way adds the splits in split order."""
    if fused_reduce is None:
        fused_reduce = num_splits == 1
    page_size = _check_paged(q, kv_cache, block_table, nkv, d)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    _check(out, "out", q.dtype)
    if rows is not None:
        _check(rows, "rows", torch.int32)
    if cluster:
        if not 2 <= num_splits <= 8:
            raise KernelError("decode_attention: a cluster takes 2 to 8 splits")
        _ok(_fn("attention_mma", "rg_decode_attention_cluster")(
            _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), _ptr(block_table), c_int(block_table.shape[1]),
            _ptr(rows), c_int(n_tokens), _ptr(req_of_token), _ptr(positions), c_int(nh), c_int(nkv), c_int(d),
            c_int(page_size), c_int(window or 0), c_float(scale), c_int(num_splits), _stream()), "decode_attention")
        return
    if scratch is None:
        part_o = torch.empty((n_tokens, nh, num_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_tokens, nh, num_splits, 2), dtype=torch.float32, device=q.device)
    else:
        part_o, part_ml = scratch
        if part_o.numel() < n_tokens * nh * num_splits * d or part_ml.numel() < n_tokens * nh * num_splits * 2:
            raise KernelError("decode_attention: the scratch buffers are too small")
    counters = None
    if fused_reduce:
        # one counter per (token, kv head, tile of 8 query heads): zero on entry, left zero by the kernel
        need = n_tokens * nkv * (-(-(nh // nkv) // 8))
        counters = _decode_counters.get(q.device)
        if counters is None or counters.numel() < need:
            counters = _decode_counters[q.device] = torch.zeros(max(need, 4096), dtype=torch.int32, device=q.device)
    else:
        _COUNTER.value += 1                  # the launcher runs two kernels: partial results, then the reduction
    _ok(_fn("attention_mma", "rg_decode_attention")(
        _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(rows), c_int(n_tokens), _ptr(req_of_token), _ptr(positions), _ptr(part_o), _ptr(part_ml),
        _ptr(counters), c_int(nh), c_int(nkv), c_int(d), c_int(page_size), c_int(window or 0), c_float(scale),
        c_int(num_splits), _stream()), "decode_attention")


_tc_err: dict = {}
TC_GEMM_MIN_ROWS = 1024        # from here the fused tcgen05 gate|up product beats cuBLAS + SiLU-mul (measured)


def tc_gemm_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Can the tcgen05 product take these operands?"""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.is_contiguous() and weight.data_ptr() % 16 == 0)


TC_TILES = {"128x128": 0, "128x256": 1, "256x256": 2, "256x128": 3}


def tc_gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype=None, silu_mul: bool = False, wide: bool = True,
            check: bool = False, tile: str | None = None) -> torch.Tensor:
    """y = x W^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor
    memory).  ``silu_mul``: W is interleaved gate|up storage and y = silu(gate)
    * up.  ``tile`` (rows of x by rows of W): "128x128" or "128x256", one CTA
    per tile, or "256x256" / "256x128", a pair of CTAs on two SMs per tile
    (cta_group::2); without it ``wide`` picks between the first two.  The
    kernel's waits are bounded; ``tc_gemm_check()`` (or ``check=True``, which
    synchronises) raises if one gave up."""
    if tile is None:
        tile = "128x256" if wide else "128x128"
    if tile not in TC_TILES:
        raise KernelError(f"tc_gemm: tile {tile!r} is not one of {sorted(TC_TILES)}")
    if not tc_gemm_ok(x, weight):
        raise KernelError(f"tc_gemm refuses x {tuple(x.shape)} {x.dtype} stride {x.stride()}, "
                          f"W {tuple(weight.shape)} {weight.dtype}: bfloat16, K a multiple of 8, 16-byte aligned")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"tc_gemm: x has {K} columns, W has {weight.shape[1]}")
    out_dtype = out_dtype or torch.bfloat16
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("tc_gemm: the SiLU-mul epilogue needs N % 16 == 0 and bfloat16 output")
    err = _tc_err.get(x.device)
    if err is None:
        err = _tc_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    global _tc_unchecked
    _tc_unchecked = True
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    _ok(_fn("gemm_tcgen05", "rg_tc_gemm")(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(out), c_int(out.shape[1]), c_int(_dtype_code(out)),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), c_int(TC_TILES[tile]), _ptr(err), _stream()),
        "tc_gemm")
    if check:
        tc_gemm_check(x.device)
    return out


TC_STREAM_MAX_ROWS = 64
# From 17 rows up to here a decode batch's layer products go through the streaming tcgen05 product with the
# neighbouring operations in its epilogues (residual addition, RMSNorm, rotation and cache write, SiLU-mul).  Alone
# the product is level with the library's; the step gains what the separate small kernels cost (measured at
# 1,024-token contexts: 10 % at batch 24, 6 % at 48, 3 % at 64).  RAILGUN_B200_TC_STREAM_ROWS overrides (16: off).
TC_STREAM_AUTO_ROWS = int(os.environ.get("RAILGUN_B200_TC_STREAM_ROWS", "64"))


def tc_stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Can the weight-streaming tcgen05 product (up to 64 rows of x) take these operands?"""
    return 0 < x.shape[0] <= TC_STREAM_MAX_ROWS and tc_gemm_ok(x, weight)


def tc_stream_gemm(x, weight: torch.Tensor, out_dtype=None, silu_mul: bool = False, splits: int = 0,
                   check: bool = False) -> torch.Tensor:
    """y = x W^T for up to 64 rows of x on the tcgen05 tensor cores with the operands swapped: 128 rows of W per
    tile stream through once, the rows of x are the narrow side.  ``silu_mul``: W is interleaved gate|up storage
    and y = silu(gate) * up.  ``splits``: 1, 2, 4 or 8 CTAs of a cluster share a tile's K and add their partial
    sums in rank order (0: as many as keep the product in one wave).  A row's result does not depend on the other
    rows.  ``x`` may be a ``NormedRows`` (an RMSNorm not finished yet): the product runs over its scaled rows and
    multiplies the 32-bit sums by 1 / rms.  The kernel's waits are bounded; ``tc_gemm_check()`` (or ``check=True``)
    raises if one gave up."""
    rows = x if isinstance(x, NormedRows) else None
    if rows is not None:
        x = rows.scaled
    if not tc_stream_ok(x, weight):
        raise KernelError(f"tc_stream_gemm refuses x {tuple(x.shape)} {x.dtype} stride {x.stride()}, "
                          f"W {tuple(weight.shape)} {weight.dtype}: bfloat16, at most 64 rows, K a multiple of 8")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"tc_stream_gemm: x has {K} columns, W has {weight.shape[1]}")
    out_dtype = out_dtype or torch.bfloat16
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("tc_stream_gemm: the SiLU-mul epilogue needs N % 16 == 0 and bfloat16 output")
    if splits not in (0, 1, 2, 4, 8) or (splits and -(-K // 64) < splits):
        raise KernelError(f"tc_stream_gemm: {splits} splits of K = {K}")
    err = _tc_err.get(x.device)
    if err is None:
        err = _tc_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    global _tc_unchecked
    _tc_unchecked = True
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    _ok(_fn("gemm_stream_tcgen05", "rg_tc_stream_gemm")(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(out), c_int(out.shape[1]), c_int(_dtype_code(out)),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), c_int(splits),
        _ptr(rows.partials if rows is not None else None), c_int(rows.blocks if rows is not None else 0),
        c_int(rows.partials.stride(0) if rows is not None else 0), c_float(rows.eps if rows is not None else 0.0),
        _ptr(err), _stream()), "tc_stream_gemm")
    if check:
        tc_gemm_check(x.device)
    return out


def tc_stream_rope_ok(x, weight: torch.Tensor, d: int) -> bool:
    """Can the q|k|v projection of these rows (17 to 64 of them) rotate and write the cache in the streaming
    tcgen05 product's own kernel?"""
    if d % 16:
        return False
    if isinstance(x, NormedRows):
        return tc_stream_scaled_ok(x, weight)
    return SKINNY_AUTO_ROWS < x.shape[0] <= TC_STREAM_AUTO_ROWS and tc_stream_ok(x, weight)


def tc_stream_gemm_rope_cache(x, weight: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, slots, kv_cache,
                              nh: int, nkv: int, d: int, err_flag=None, splits: int = 0) -> torch.Tensor:
    """``skinny_gemm_rope_cache`` for up to 64 rows: the q|k|v projection with the rotary encoding and the cache
    write in the product's epilogue.  Returns [M, (nh+2nkv)d] whose q heads are rotated (its k and v columns are
    not written); k (rotated) and v go to ``kv_cache`` at ``slots`` (None: no write).  ``x``: bfloat16 rows or a
    ``NormedRows``; ``weight``'s q and k rows are in ``rope_pair_order``."""
    rows = x if isinstance(x, NormedRows) else None
    xin = rows.scaled if rows is not None else x
    if d % 16 or not tc_stream_ok(xin, weight):
        raise KernelError(f"tc_stream_gemm_rope_cache refuses rows {tuple(xin.shape)}, W {tuple(weight.shape)}, head size {d}")
    M, K = xin.shape
    N = weight.shape[0]
    if weight.shape[1] != K or N != (nh + 2 * nkv) * d:
        raise KernelError(f"tc_stream_gemm_rope_cache: W {tuple(weight.shape)} is not [({nh} + 2 x {nkv}) x {d}, {K}]")
    _check(table, "rope table", torch.float32)
    _check(positions, "positions", torch.int32)
    if table.shape[1] != d or positions.numel() < M:
        raise KernelError("tc_stream_gemm_rope_cache: the table's head size or the number of positions does not match")
    page_size = 0
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", torch.bfloat16)
        page_size = kv_cache.shape[3]
        if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d) or slots.numel() < M:
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match [pages, 2, {nkv}, page, {d}]")
    err = _tc_err.get(xin.device)
    if err is None:
        err = _tc_err[xin.device] = torch.zeros(1, dtype=torch.int32, device=xin.device)
    global _tc_unchecked
    _tc_unchecked = True
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xin.device)
    _ok(_fn("gemm_stream_tcgen05", "rg_tc_stream_gemm_rope_cache")(
        _ptr(xin), c_int(xin.stride(0)), _ptr(weight), _ptr(out), c_int(N), c_int(M), c_int(N), c_int(K), c_int(splits),
        _ptr(rows.partials if rows is not None else None), c_int(rows.blocks if rows is not None else 0),
        c_int(rows.partials.stride(0) if rows is not None else 0), c_float(rows.eps if rows is not None else 0.0),
        _ptr(table), _ptr(positions), _ptr(slots), _ptr(kv_cache if slots is not None else None), c_int(nh), c_int(nkv),
        c_int(d), c_int(page_size), c_int(table.shape[0]), _ptr(err_flag), _ptr(err), _stream()),
        "tc_stream_gemm_rope_cache")
    return out


def tc_stream_fused_ok(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor) -> bool:
    """Can x W^T be added to ``resid`` inside the streaming tcgen05 product (which then also prepares the next
    norm)?  Decode batches above the skinny product's and up to ``TC_STREAM_AUTO_ROWS`` rows."""
    return (SKINNY_AUTO_ROWS < x.shape[0] <= TC_STREAM_AUTO_ROWS and tc_stream_ok(x, weight)
            and resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == (x.shape[0], weight.shape[0])
            and resid.shape[1] % 8 == 0)


def tc_stream_gemm_residual(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor,
                            eps: float, splits: int = 0) -> NormedRows:
    """resid += x W^T (32-bit, in place), and the RMSNorm (``norm_weight``, ``eps``) of the new rows but for the
    factor 1 / rms, which the product that reads the result applies (``skinny_gemm_residual`` for 17 to 64 rows)."""
    if not tc_stream_ok(x, weight):
        raise KernelError(f"tc_stream_gemm_residual refuses x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)}")
    _check(resid, "resid", torch.float32)
    _check(norm_weight, "norm_weight", torch.float32)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or resid.shape != (M, N) or norm_weight.numel() != N:
        raise KernelError(f"tc_stream_gemm_residual: x {tuple(x.shape)}, W {tuple(weight.shape)}, residual "
                          f"{tuple(resid.shape)}, norm weight {norm_weight.numel()}")
    partials = torch.empty((-(-N // 128), TC_STREAM_MAX_ROWS), dtype=torch.float32, device=x.device)
    scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    err = _tc_err.get(x.device)
    if err is None:
        err = _tc_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    global _tc_unchecked
    _tc_unchecked = True
    tiles = c_int(0)
    _ok(_fn("gemm_stream_tcgen05", "rg_tc_stream_gemm_residual")(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(resid), c_int(resid.stride(0)), _ptr(norm_weight), _ptr(scaled),
        _ptr(partials), c_int(partials.stride(0)), c_int(M), c_int(N), c_int(K), c_int(splits), ctypes.byref(tiles),
        _ptr(err), _stream()), "tc_stream_gemm_residual")
    return NormedRows(resid, scaled, partials, tiles.value, norm_weight, eps, torch.bfloat16)


def tc_stream_scaled_ok(rows: NormedRows, weight: torch.Tensor) -> bool:
    return (rows.dtype == torch.bfloat16 and SKINNY_AUTO_ROWS < rows.shape[0] <= TC_STREAM_AUTO_ROWS
            and tc_stream_ok(rows.scaled, weight) and rows.shape[1] == weight.shape[1])


_tc_unchecked = False


def mark_tc_unchecked() -> None:
    """A replayed graph may have run tcgen05 kernels: the next ``tc_gemm_check`` looks at their error flag."""
    global _tc_unchecked
    _tc_unchecked = True


def prefill_attention_tc_ok(q, kv_cache, d: int, page_size: int) -> bool:
    """Can the tcgen05 flash kernel take this?  bfloat16, head size 64, pages of 8, 16, 32, 64 or 128 tokens."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and d == 64 and page_size in (8, 16, 32, 64, 128)
            and q.dim() == 2 and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and kv_cache.is_contiguous())


def prefill_attention_tc(q, out, kv_cache, block_table, tiles, positions, nh: int, nkv: int, d: int,
                         window: int, scale: float) -> None:
    """Flash attention on the tcgen05 tensor cores for requests that bring
    several tokens: ``q`` is the fused qkv buffer [T, (nh + 2 nkv) d], ``tiles``
    [n, 3] = (first row, rows <= 128, request index).  Writes the tiles' rows
    of ``out`` [T, nh*d].  Its waits are bounded; ``tc_gemm_check()`` raises if
    one gave up."""
    page_size = kv_cache.shape[3]
    if not prefill_attention_tc_ok(q, kv_cache, d, page_size):
        raise KernelError("prefill_attention_tc: bfloat16, head size 64, page size 8..128 dividing 128")
    _check(kv_cache, "kv_cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    _check(tiles, "tiles", torch.int32)
    _check(positions, "positions", torch.int32)
    _check(out, "out", q.dtype)
    if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match heads {nkv} x {d}")
    err = _tc_err.get(q.device)
    if err is None:
        err = _tc_err[q.device] = torch.zeros(1, dtype=torch.int32, device=q.device)
    global _tc_unchecked
    _tc_unchecked = True
    _ok(_fn("attention_tcgen05", "rg_prefill_attention_tc")(
        _ptr(q), c_int(q.stride(0)), c_int(q.shape[0]), _ptr(out), _ptr(kv_cache), c_int(kv_cache.shape[0]),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(tiles), c_int(tiles.shape[0]), _ptr(positions),
        c_int(nh), c_int(nkv), c_int(d), c_int(page_size), c_int(window or 0), c_float(scale), _ptr(err),
        _stream()), "prefill_attention_tc")


def probe_sm100(device="cuda:0") -> dict:
    """Cycle counts of the building blocks of the tcgen05 kernels on this GPU
    (csrc/kernels/probe_sm100.cu): a diagnostic, on no product path."""
    from ctypes import c_double
    names = ["ex2.approx.ftz.f32", "cvt.rn.bf16x2.f32", "fma.rn.f32x2", "fma.rn.f32", "max.f32",
             "tcgen05.mma M128 N64 K16", "tcgen05.mma M128 N128 K16", "tcgen05.mma M128 N256 K16",
             "four N64 MMAs + two commits", "mbarrier wait (done), every lane", "mbarrier wait (done), lane 0 + shuffle",
             "fence.proxy.async", "mbarrier.arrive", "tcgen05.st x8 + wait::st",
             "softmax pass of 64 columns, 2 warps per scheduler", "softmax pass of 64 columns, 1 warp per scheduler"]
    dev = torch.device(device)
    scratch = torch.randn(148 * 512 * 64, device=dev)
    cyc = torch.zeros(16, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out = (c_double * len(names))()
    with torch.cuda.device(dev):
        _ok(_fn("probe_sm100", "rg_probe_sm100")(out, _ptr(scratch), _ptr(cyc), _ptr(err), _stream()), "probe_sm100")
    if int(err.item()) != 0 or any(v < 0 for v in out):
        raise KernelError(f"probe_sm100: a bounded wait gave up (code {int(err.item())})")
    return {n: round(float(v), 1) for n, v in zip(names, out)}


def tc_gemm_check(device=None) -> None:
    """Raise if a wait inside a tcgen05 product gave up since the last check
    (synchronises; free when no such product ran since)."""
    global _tc_unchecked
    if not _tc_unchecked:
        return
    _tc_unchecked = False
    for dev, err in _tc_err.items():
        if device is not None and dev != device:
            continue
        code = int(err.item())
        if code:
            err.zero_()
            who = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue", 4: "the MMA issuer"}.get(
                code, f"role {code} of the attention kernel")
            raise KernelError(f"a tcgen05 kernel: {who} gave up waiting on a barrier; the result is invalid")


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of every row, ties to the lowest index
    (into ``out``, int32 [rows], if given)."""
    _check(logits, "logits", torch.float32)
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _check(out, "out", torch.int32)
        if out.shape != (rows,):
            raise KernelError(f"argmax: out has shape {tuple(out.shape)}, the logits have {rows} rows")
    pieces = min(64, -(-V // 2048))            # wide rows are cut into pieces so that many blocks share a row
    pv = pi = None
    if pieces > 1:
        pv = torch.empty((rows, pieces), dtype=torch.float32, device=logits.device)
        pi = torch.empty((rows, pieces), dtype=torch.int32, device=logits.device)
        _COUNTER.value += 1
    _ok(_fn("sampling", "rg_argmax")(_ptr(logits), c_int(rows), c_int(V), _ptr(out), _ptr(pv), _ptr(pi),
                                     c_int(pieces), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k, top_p, seed: torch.Tensor,
           counter: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row; rows with temperature <= 0 are greedy.  ``seed`` and
    ``counter`` are int64 tensors read as unsigned 64-bit."""
    _check(logits, "logits", torch.float32)
    rows, V = logits.shape
    _check(temperature, "temperature", torch.float32)
    _check(seed, "seed", torch.int64)
    _check(counter, "counter", torch.int64)
    if top_k is not None:
        _check(top_k, "top_k", torch.int32)
    if top_p is not None:
        _check(top_p, "top_p", torch.float32)
    for name, t in (("temperature", temperature), ("seed", seed), ("counter", counter),
                    ("top_k", top_k), ("top_p", top_p)):
        if t is not None and t.numel() != rows:
            raise KernelError(f"{name} has {t.numel()} entries for {rows} rows")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _check(out, "out", torch.int32)
        if out.shape != (rows,):
            raise KernelError(f"sample: out has shape {tuple(out.shape)}, the logits have {rows} rows")
    _ok(_fn("sampling", "rg_sample")(_ptr(logits), c_int(rows), c_int(V), _ptr(temperature), _ptr(top_k),
                                     _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out), _stream()), "sample")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """y = x W^T, W stored [out, in].  Up to 64 bfloat16 rows go through the
    weight-streaming kernel of this package; everything else through the
    library matrix product (cuBLAS), as in the reference, whose projections
    are library GEMMs (crates/vllm-models/src/llama/attention.rs:94-96,133).
    32-bit inputs run in true 32-bit: the reduced-precision matrix mode is
    refused."""
    if isinstance(x, NormedRows):
        if (out_dtype is None or out_dtype == torch.bfloat16) and skinny_scaled_ok(x, weight):
            return skinny_gemm_scaled(x, weight)              # the norm is finished inside the product
        if tc_stream_scaled_ok(x, weight):
            return tc_stream_gemm(x, weight, out_dtype)      # likewise, for 17 to 64 rows
        x = x.materialize()
    if not x.is_cuda:
        raise KernelError("linear: CUDA tensors only (there is no CPU path)")
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("linear: TF32 is enabled; the 32-bit path must be true 32-bit")
    if x.shape[0] <= SKINNY_AUTO_ROWS and skinny_gemm_ok(x, weight):
        return skinny_gemm(x, weight, out_dtype)             # small decode batches: stream the weights once
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    return torch.mm(x, weight.t())

