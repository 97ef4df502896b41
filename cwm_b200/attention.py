"""Paged-KV grouped-query attention and the fused rotate + cache-write step.

``mha_fwd`` keeps the signature with which ``cwm/fastgen/forward.py:639-655``
calls ``xformers.ops.fmha.flash3.mha_fwd``; ``rope_kv_write`` does in one launch
what ``forward.py:618-632`` does in four (two ``apply_rope`` and two
``paged_memcpy`` calls).
"""

from __future__ import annotations

import torch

from . import _lib
from .kernels import _DTYPES, _on_device, _ptr, _require_cuda, _stream, _use_registered_op

_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_capture_workspaces: dict[int, torch.Tensor] = {}
# problem size the cached workspace is sized for; larger ones get a fresh one
_WS_BATCH_X_HEADS = 16384 * 8


def _new_workspace(device: torch.device, batch: int, hkv: int) -> torch.Tensor:
    need = _lib.load().cwm_paged_attn_workspace_bytes(batch, 0, 0, hkv, 0)
    # zero-filled once: the arrival counters in it must start at zero, and every
    # call leaves them zero
    return torch.zeros(need, dtype=torch.uint8, device=device)


def workspace_for(device: torch.device, batch: int, hkv: int = 8) -> torch.Tensor:
    """Scratch buffer for ``mha_fwd`` on ``device`` (arrival counters and split-KV
    partial results of the decode kernel).

    Eager calls share one buffer per device and stream, which is safe because calls
    on one stream run in order.  Calls made while a CUDA graph is being captured use
    a second, per-device buffer that is allocated (and cleared) by the first eager
    call on that device, outside any graph pool, and is never dropped: every graph
    captured on the device points at it, so graphs must not be replayed
    concurrently with each other.  A capture on a device that has not seen an eager
    call yet takes a fresh buffer from the graph's pool for every call instead,
    cleared by a memset node on each replay.
    """
    index = device.index if device.index is not None else torch.cuda.current_device()
    fits = batch * hkv <= _WS_BATCH_X_HEADS
    if torch.cuda.is_current_stream_capturing():
        ws = _capture_workspaces.get(index)
        if ws is not None and fits:
            return ws
        return _new_workspace(device, batch, hkv)
    if index not in _capture_workspaces:
        _capture_workspaces[index] = _new_workspace(device, _WS_BATCH_X_HEADS // 8, 8)
    key = (index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if fits:
        if ws is None:
            ws = _new_workspace(device, _WS_BATCH_X_HEADS // 8, 8)
            _workspaces[key] = ws
        return ws
    need = _lib.load().cwm_paged_attn_workspace_bytes(batch, 0, 0, hkv, 0)
    if ws is None or ws.numel() < need:
        ws = _new_workspace(device, batch, hkv)
        _workspaces[key] = ws
    return ws


def reset_workspaces() -> None:
    """Clear the arrival counters of every cached workspace (a call that ended with
    a device status word other than 0 may have left them non-zero)."""
    # a workspace made inside torch.inference_mode() may only be written in that mode
    with torch.inference_mode():
        for ws in list(_workspaces.values()) + list(_capture_workspaces.values()):
            ws.zero_()


_lib.on_bad_status.append(reset_workspaces)


def _paged_attn_launch(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    seqused_k: torch.Tensor,
    block_table: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: float,
    window_left: int,
    out: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    total_q, hq, d = query.shape
    num_pages, page_size, hkv, _ = key.shape
    batch = seqused_k.shape[0]
    if out is None:
        out = torch.empty_like(query)
    lse = torch.empty((hq, total_q), dtype=torch.float32, device=query.device)
    if total_q == 0 or batch == 0:
        return out, lse
    ws = workspace_for(query.device, batch, hkv)
    with _on_device(query):
        code = _lib.load().cwm_paged_attn_fwd(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), lse.data_ptr(),
            cu_seqlens_q.data_ptr(), seqused_k.data_ptr(), block_table.data_ptr(), batch,
            total_q, hq, hkv, d, _DTYPES[query.dtype], page_size, num_pages, key.stride(1),
            block_table.stride(0), max_seqlen_q, max_seqlen_k, softmax_scale, window_left,
            ws.data_ptr(), ws.numel(), _stream(query),
        )
    _lib.check(code, "mha_fwd")
    return out, lse


def _paged_attn_impl(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    seqused_k: torch.Tensor,
    block_table: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: float,
    window_left: int,
) -> tuple[torch.Tensor, torch.Tensor]:
    return _paged_attn_launch(query, key, value, cu_seqlens_q, seqused_k, block_table,
                              max_seqlen_q, max_seqlen_k, softmax_scale, window_left)


_paged_attn_op = torch.library.custom_op(
    "cwm_b200::paged_attn_fwd", mutates_args=(), device_types="cuda")(_paged_attn_impl)


@_paged_attn_op.register_fake
def _(query, key, value, cu_seqlens_q, seqused_k, block_table, max_seqlen_q, max_seqlen_k,
      softmax_scale, window_left):
    return torch.empty_like(query), query.new_empty(
        (query.shape[1], query.shape[0]), dtype=torch.float32
    )


def mha_fwd(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor | None,
    seqused_k: torch.Tensor,
    leftpad_k: torch.Tensor | None,
    max_seqlen_q: int,
    max_seqlen_k: int,
    p: float,
    block_table: torch.Tensor,
    softmax_scale: float,
    is_causal: bool = True,
    window_left: int = -1,
    window_right: int = -1,
    out: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Variable-length paged grouped-query attention forward.

    Same arguments as the call at ``cwm/fastgen/forward.py:639-655``:

    * ``query``: ``(T, Hq, 128)`` contiguous, bf16 or fp16;
    * ``key``, ``value``: ``(pages, page_size, Hkv, 128)`` views of the cache rows
      (``cache_k.reshape(-1, page_size, Hkv, 128)``): unit stride in the last
      dimension, heads contiguous, any token stride;
    * ``cu_seqlens_q``: int32 ``(B + 1,)`` query offsets; ``seqused_k``: int32
      ``(B,)`` keys per sequence (including the queries' own tokens);
    * ``block_table``: int32 ``(B, cols)``, row stride free;
    * ``max_seqlen_q`` / ``max_seqlen_k``: static upper bounds (in graph-captured
      decode ``max_seqlen_k`` is the cache capacity of a lane, not the true
      maximum);
    * ``window_left``: keys further than this to the left of the query are
      masked; negative means unbounded.

    Only what the reference uses is built: ``cu_seqlens_k`` and ``leftpad_k`` must
    be None, ``p`` 0, ``is_causal`` True and ``window_right`` -1 or 0.

    ``out`` (not in the reference's signature): where to write the result instead
    of a new tensor; contiguous, shaped and typed like ``query``, on the device or in
    pinned host memory (the kernels then store the rows straight across the host
    link, which saves the separate device-to-host copy of a step's output).

    Returns ``(out, lse)`` with ``out`` like ``query`` and ``lse`` float32
    ``(Hq, T)``.
    """
    if cu_seqlens_k is not None or leftpad_k is not None:
        raise ValueError("cu_seqlens_k and leftpad_k are not supported (pass None)")
    if p != 0:
        raise ValueError("dropout is not supported (p must be 0)")
    if not is_causal or window_right not in (-1, 0):
        raise ValueError("only causal attention (is_causal=True, window_right=-1) is supported")
    if query.ndim != 3:
        raise ValueError(f"query must be (T, Hq, D), got {query.ndim}-D")
    if key.ndim != 4 or value.ndim != 4 or key.shape != value.shape:
        raise ValueError("key and value must be (pages, page_size, Hkv, D) with equal shapes")
    if query.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"query must be bf16 or fp16, got {query.dtype}")
    if key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError("query, key and value must share a dtype")
    if not query.is_contiguous():
        raise ValueError("query must be contiguous")
    _, hq, d = query.shape
    _, page_size, hkv, dk = key.shape
    if dk != d:
        raise ValueError(f"head dimensions differ: query {d}, key {dk}")
    if hkv == 0 or hq % hkv != 0:
        raise ValueError(f"{hq} query heads cannot be grouped over {hkv} KV heads")
    for name, t in (("key", key), ("value", value)):
        if t.stride(3) != 1 or (hkv > 1 and t.stride(2) != d):
            raise ValueError(f"{name} must keep heads contiguous within a token row")
        if t.shape[0] > 1 and t.stride(0) != page_size * t.stride(1):
            raise ValueError(f"{name} pages must be consecutive row ranges of the cache")
    if key.stride(1) != value.stride(1):
        raise ValueError("key and value must have the same token stride")
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("seqused_k", seqused_k)):
        if t.dtype != torch.int32 or t.ndim != 1 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous 1-D int32 tensor")
    batch = seqused_k.shape[0]
    if cu_seqlens_q.shape[0] != batch + 1:
        raise ValueError(f"cu_seqlens_q must have {batch + 1} entries, got {cu_seqlens_q.shape[0]}")
    if block_table.dtype != torch.int32 or block_table.ndim != 2:
        raise ValueError("block_table must be a 2-D int32 tensor")
    if block_table.shape[0] < batch:
        raise ValueError("block_table has fewer rows than sequences")
    if block_table.shape[1] > 1 and block_table.stride(1) != 1:
        raise ValueError("block_table must have unit stride in its last dimension")
    _require_cuda("mha_fwd", query, key, value, cu_seqlens_q, seqused_k, block_table)
    # never read past the block table, whatever bound the caller gave
    max_k = min(int(max_seqlen_k), block_table.shape[1] * page_size)
    if out is not None:
        if (out.shape != query.shape or out.dtype != query.dtype or not out.is_contiguous()
                or not (out.is_cuda or out.is_pinned())):
            raise ValueError("out must be contiguous, shaped and typed like query, and live on "
                             "the device or in pinned host memory")
        return _paged_attn_launch(query, key, value, cu_seqlens_q, seqused_k, block_table,
                                  int(max_seqlen_q), max_k, float(softmax_scale),
                                  int(window_left), out)
    return (_paged_attn_op if _use_registered_op() else _paged_attn_impl)(
        query, key, value, cu_seqlens_q, seqused_k, block_table, int(max_seqlen_q), max_k,
        float(softmax_scale), int(window_left),
    )


def _rope_kv_write_impl(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    pos: torch.Tensor,
    freqs: torch.Tensor,
    page_tbl: torch.Tensor,
    src_batch: torch.Tensor | None,
    batch_size: torch.Tensor | None,
    page_size: int,
) -> None:
    t, hq, d = xq.shape
    hkv = xk.shape[1]
    with _on_device(xq):
        code = _lib.load().cwm_rope_kv_write(
            xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
            pos.data_ptr(), freqs.data_ptr(), page_tbl.data_ptr(), _ptr(src_batch),
            _ptr(batch_size), int(batch_size is not None and batch_size.dtype == torch.int64),
            t, hq, hkv, d, _DTYPES[xq.dtype], page_size, page_tbl.stride(0), page_tbl.shape[1],
            cache_k.stride(0), cache_k.shape[0], _stream(xq),
        )
    _lib.check(code, "rope_kv_write")


_rope_kv_write_op = torch.library.custom_op(
    "cwm_b200::rope_kv_write", mutates_args=("xq", "xk", "cache_k", "cache_v"),
    device_types="cuda")(_rope_kv_write_impl)


def rope_kv_write(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    pos: torch.Tensor,
    freqs: torch.Tensor,
    page_tbl: torch.Tensor,
    src_batch: torch.Tensor | None,
    batch_size: torch.Tensor | None,
    page_size: int,
) -> None:
    """Rotate ``xq`` and ``xk`` in place and store the rotated ``xk`` and ``xv``
    rows in their pages, in one launch.

    Equivalent to the sequence at ``cwm/fastgen/forward.py:618-632``::

        apply_rope(xq, pos, freqs); apply_rope(xk, pos, freqs)
        paged_memcpy(xk.flatten(1, 2), cache_k, page_tbl, pos, None, src_batch, batch_size, P)
        paged_memcpy(xv.flatten(1, 2), cache_v, page_tbl, pos, None, src_batch, batch_size, P)

    ``xq``: ``(T, Hq, D)``; ``xk``, ``xv``: ``(T, Hkv, D)``; ``cache_k``/``cache_v``:
    the two column halves of a cache layer as returned by ``RawCache.cache_kv``.
    Rows at or beyond ``batch_size`` are rotated but not stored, as in the
    reference.
    """
    if xq.ndim != 3 or xk.ndim != 3 or xv.ndim != 3:
        raise ValueError("xq, xk and xv must be 3-D (T, H, D)")
    t, _, d = xq.shape
    if xk.shape[0] != t or xv.shape != xk.shape or xk.shape[2] != d:
        raise ValueError("xq, xk and xv disagree on the token count or head dimension")
    if not (xq.is_contiguous() and xk.is_contiguous() and xv.is_contiguous()):
        raise ValueError("xq, xk and xv must be contiguous")
    if not (xq.dtype == xk.dtype == xv.dtype == cache_k.dtype == cache_v.dtype):
        raise ValueError("xq, xk, xv and the cache must share a dtype")
    if xq.dtype not in _DTYPES:
        raise ValueError(f"dtype {xq.dtype} is not supported")
    hkv = xk.shape[1]
    for name, c in (("cache_k", cache_k), ("cache_v", cache_v)):
        if c.ndim != 2 or c.shape[1] != hkv * d or c.stride(1) != 1:
            raise ValueError(f"{name} must be (rows, Hkv * D) with unit stride in its last dimension")
    if cache_k.stride(0) != cache_v.stride(0) or cache_k.shape[0] != cache_v.shape[0]:
        raise ValueError("cache_k and cache_v must be halves of the same cache rows")
    if pos.dtype != torch.int32 or pos.ndim != 1 or pos.shape[0] != t or not pos.is_contiguous():
        raise ValueError(f"pos must be a contiguous int32 tensor of shape ({t},)")
    if freqs.dtype != torch.float32 or freqs.ndim != 1 or freqs.shape[0] * 2 != d:
        raise ValueError(f"freqs must be a float32 tensor of shape ({d // 2},)")
    if not freqs.is_contiguous():
        raise ValueError("freqs must be contiguous")
    if page_tbl.dtype != torch.int32 or page_tbl.ndim != 2:
        raise ValueError("page_tbl must be a 2-D int32 tensor")
    if page_tbl.shape[1] > 1 and page_tbl.stride(1) != 1:
        raise ValueError("page_tbl must have unit stride in its last dimension")
    if src_batch is not None:
        if (src_batch.dtype != torch.int32 or src_batch.ndim != 1 or src_batch.shape[0] != t
                or not src_batch.is_contiguous()):
            raise ValueError(f"src_batch must be a contiguous int32 tensor of shape ({t},)")
    if batch_size is not None:
        if batch_size.ndim != 0 or batch_size.dtype not in (torch.int32, torch.int64):
            raise ValueError("batch_size must be a 0-d int32 or int64 tensor")
        if src_batch is not None:
            raise ValueError("src_batch and batch_size cannot be given together")
    _require_cuda("rope_kv_write", xq, xk, xv, cache_k, cache_v, pos, freqs, page_tbl,
                  src_batch, batch_size)
    fn = _rope_kv_write_op if _use_registered_op() else _rope_kv_write_impl
    fn(xq, xk, xv, cache_k, cache_v, pos, freqs, page_tbl, src_batch, batch_size, page_size)


def qkv_rope_kv_write(
    qkv: torch.Tensor,
    n_heads: int,
    n_kv_heads: int,
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    pos: torch.Tensor,
    freqs: torch.Tensor,
    page_tbl: torch.Tensor,
    src_batch: torch.Tensor | None,
    batch_size: torch.Tensor | None,
    page_size: int,
) -> torch.Tensor:
    """``rope_kv_write`` for a runner that computes the q, k and v projections as one
    product: ``qkv`` is ``(T, (Hq + 2 Hkv) * D)`` with rows ``[q heads | k heads | v
    heads]`` (any row stride).  Returns the rotated queries ``(T, Hq, D)``; the
    rotated keys and the values go straight to their pages, ``qkv`` is only read.
    Same positions, block table and ``batch_size`` rule as ``rope_kv_write``
    (``cwm/fastgen/forward.py:608-632``).  ``qkv`` may also live in pinned host
    memory: the kernel then reads the rows straight across the host link, which
    saves the separate host-to-device copy of a step's inputs."""
    if qkv.ndim != 2 or qkv.stride(1) != 1:
        raise ValueError("qkv must be 2-D (T, (Hq + 2 Hkv) * D) with unit stride in its last dimension")
    t, width = qkv.shape
    heads = n_heads + 2 * n_kv_heads
    if heads <= 0 or width % heads != 0:
        raise ValueError(f"qkv rows of {width} elements do not hold {heads} heads")
    d = width // heads
    if qkv.dtype not in _DTYPES or cache_k.dtype != qkv.dtype or cache_v.dtype != qkv.dtype:
        raise ValueError("qkv and the cache must share a supported dtype")
    for name, c in (("cache_k", cache_k), ("cache_v", cache_v)):
        if c.ndim != 2 or c.shape[1] != n_kv_heads * d or c.stride(1) != 1:
            raise ValueError(f"{name} must be (rows, Hkv * D) with unit stride in its last dimension")
    if cache_k.stride(0) != cache_v.stride(0) or cache_k.shape[0] != cache_v.shape[0]:
        raise ValueError("cache_k and cache_v must be halves of the same cache rows")
    if pos.dtype != torch.int32 or pos.shape != (t,) or not pos.is_contiguous():
        raise ValueError(f"pos must be a contiguous int32 tensor of shape ({t},)")
    if freqs.dtype != torch.float32 or freqs.shape != (d // 2,) or not freqs.is_contiguous():
        raise ValueError(f"freqs must be a contiguous float32 tensor of shape ({d // 2},)")
    if page_tbl.dtype != torch.int32 or page_tbl.ndim != 2 or (
            page_tbl.shape[1] > 1 and page_tbl.stride(1) != 1):
        raise ValueError("page_tbl must be a 2-D int32 tensor with unit stride in its last dimension")
    if src_batch is not None and (src_batch.dtype != torch.int32 or src_batch.shape != (t,)
                                  or not src_batch.is_contiguous()):
        raise ValueError(f"src_batch must be a contiguous int32 tensor of shape ({t},)")
    if batch_size is not None:
        if batch_size.ndim != 0 or batch_size.dtype not in (torch.int32, torch.int64):
            raise ValueError("batch_size must be a 0-d int32 or int64 tensor")
        if src_batch is not None:
            raise ValueError("src_batch and batch_size cannot be given together")
    if not qkv.is_cuda and not qkv.is_pinned():
        raise RuntimeError("qkv_rope_kv_write: qkv must live on a CUDA device or in pinned host "
                           "memory")
    _require_cuda("qkv_rope_kv_write", cache_k, cache_v, pos, freqs, page_tbl, src_batch,
                  batch_size)
    q_out = torch.empty((t, n_heads, d), dtype=qkv.dtype, device=cache_k.device)
    with _on_device(cache_k):
        code = _lib.load().cwm_qkv_rope_kv_write(
            qkv.data_ptr(), qkv.stride(0) if t > 1 else width, q_out.data_ptr(),
            cache_k.data_ptr(), cache_v.data_ptr(), pos.data_ptr(), freqs.data_ptr(),
            page_tbl.data_ptr(), _ptr(src_batch), _ptr(batch_size),
            int(batch_size is not None and batch_size.dtype == torch.int64), t, n_heads,
            n_kv_heads, d, _DTYPES[qkv.dtype], page_size, page_tbl.stride(0), page_tbl.shape[1],
            cache_k.stride(0), cache_k.shape[0], _stream(cache_k),
        )
    _lib.check(code, "qkv_rope_kv_write")
    return q_out


def silu_mul(x13: torch.Tensor) -> torch.Tensor:
    """``F.silu(x1, inplace=True).mul_(x3)`` (``cwm/fastgen/forward.py:776-781``) for
    the stacked product ``x13 = [x1 | x3]`` of shape ``(T, 2 * ffn)``, in one launch;
    returns ``(T, ffn)``."""
    if x13.ndim != 2 or x13.shape[1] % 2 != 0 or not x13.is_contiguous():
        raise ValueError("x13 must be a contiguous 2-D tensor (T, 2 * ffn)")
    if x13.dtype not in _DTYPES:
        raise ValueError(f"dtype {x13.dtype} is not supported")
    _require_cuda("silu_mul", x13)
    t, ffn = x13.shape[0], x13.shape[1] // 2
    out = torch.empty((t, ffn), dtype=x13.dtype, device=x13.device)
    with _on_device(x13):
        code = _lib.load().cwm_silu_mul(x13.data_ptr(), out.data_ptr(), t, ffn,
                                        _DTYPES[x13.dtype], _stream(x13))
    _lib.check(code, "silu_mul")
    return out
