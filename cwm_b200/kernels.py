"""Drop-in replacements for ``cwm/fastgen/kernels`` (``apply_rope``,
``paged_memcpy``, ``rmsnorm``), backed by hand-written sm_100a kernels.

Signatures, argument meaning and error behaviour follow the reference: argument
problems raise ``ValueError`` before anything is launched
(``kernels/rope.py:117-140``, ``kernels/paged_memcpy.py:143-211``,
``kernels/rmsnorm.py:88-102``).  Each function validates on the host and then
dispatches to a PyTorch custom op (``torch.ops.cwm_b200.*``) that calls the C ABI
on torch's current stream, so the ops can be captured in CUDA graphs.
"""

from __future__ import annotations

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.CWM_BF16, torch.float16: _lib.CWM_F16, torch.float32: _lib.CWM_F32}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on_device(t: torch.Tensor):
    """Context that makes ``t``'s device current for the C-ABI call; free when it
    already is (the usual one-process-per-GPU case)."""
    if t.device.index is None or t.device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(t.device)


def _dtype_code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"{what}: dtype {t.dtype} is not supported") from None


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require_cuda(what: str, *tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                f"{what}: tensors must live on a CUDA device (there is no CPU implementation)"
            )


# ----------------------------------------------------------------- custom ops
# Each op exists twice: as a plain function that calls the C ABI, and registered as
# ``torch.ops.cwm_b200.*`` (schema, mutation annotations, fake implementation) for
# code that is traced or compiled.  In eager mode, CUDA-graph capture included, the
# public wrappers call the plain function: the dispatcher adds tens of microseconds
# per call and nothing that eager execution needs.
def _use_registered_op() -> bool:
    return torch.compiler.is_compiling()



def _rope_impl(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor) -> None:
    n, h, d = x.shape
    with _on_device(x):
        code = _lib.load().cwm_rope(
            x.data_ptr(), pos.data_ptr(), freqs.data_ptr(), n, h, d, _DTYPES[x.dtype], _stream(x)
        )
    _lib.check(code, "apply_rope")


_rope_op = torch.library.custom_op(
    "cwm_b200::rope", mutates_args=("x",), device_types="cuda")(_rope_impl)


def _rmsnorm_impl(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    out = torch.empty_like(x)
    n, d = x.shape
    with _on_device(x):
        code = _lib.load().cwm_rmsnorm(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), n, d, eps, _DTYPES[x.dtype], _stream(x)
        )
    _lib.check(code, "rmsnorm")
    return out


_rmsnorm_op = torch.library.custom_op(
    "cwm_b200::rmsnorm", mutates_args=(), device_types="cuda")(_rmsnorm_impl)


@_rmsnorm_op.register_fake
def _(x, w, eps):
    return torch.empty_like(x)


def _add_rmsnorm_impl(h: torch.Tensor, delta: torch.Tensor, w: torch.Tensor,
                    eps: float) -> torch.Tensor:
    out = torch.empty_like(h)
    n, d = h.shape
    with _on_device(h):
        code = _lib.load().cwm_add_rmsnorm(
            h.data_ptr(), delta.data_ptr(), w.data_ptr(), out.data_ptr(), n, d, eps,
            _DTYPES[h.dtype], _stream(h),
        )
    _lib.check(code, "add_rmsnorm")
    return out


_add_rmsnorm_op = torch.library.custom_op(
    "cwm_b200::add_rmsnorm", mutates_args=("h",), device_types="cuda")(_add_rmsnorm_impl)


@_add_rmsnorm_op.register_fake
def _(h, delta, w, eps):
    return torch.empty_like(h)


def _paged_memcpy_impl(
    src: torch.Tensor,
    dst: torch.Tensor,
    page_tbl: torch.Tensor,
    dst_pos: torch.Tensor,
    shard_idx: int,
    shard_cnt: int,
    src_batch: torch.Tensor | None,
    batch_size: torch.Tensor | None,
    page_size: int,
) -> None:
    n, e = src.shape
    with _on_device(src):
        code = _lib.load().cwm_paged_memcpy(
            src.data_ptr(), dst.data_ptr(), page_tbl.data_ptr(), dst_pos.data_ptr(),
            _ptr(src_batch), _ptr(batch_size),
            int(batch_size is not None and batch_size.dtype == torch.int64),
            n, e, src.element_size(), page_size, page_tbl.stride(0), page_tbl.shape[1],
            dst.stride(0), dst.shape[0], shard_idx, shard_cnt, _stream(src),
        )
    _lib.check(code, "paged_memcpy")


_paged_memcpy_op = torch.library.custom_op(
    "cwm_b200::paged_memcpy", mutates_args=("dst",), device_types="cuda")(_paged_memcpy_impl)


# ------------------------------------------------------------ public wrappers
def apply_rope(
    x: torch.Tensor,
    pos: torch.Tensor,
    freqs: torch.Tensor,
    approx_trigo: bool = False,
) -> None:
    """Rotate ``x`` in place (``cwm/fastgen/kernels/rope.py:93-163``).

    ``x``: ``(N, H, D)`` contiguous; ``pos``: int32 ``(N,)``; ``freqs``: float32
    ``(D/2,)``.  Pair ``i`` of a head is ``(x[2i], x[2i+1])``; the math is fp32
    with the angle ``float32(pos) * freqs[i]``.  ``approx_trigo`` is accepted for
    signature compatibility; the accurate sine and cosine are always used (no
    caller of the reference enables the approximation).
    """
    if x.ndim != 3:
        raise ValueError(f"x must have 3 dimensions (N, H, D), got {x.ndim}")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    n, _, d = x.shape
    if pos.ndim != 1 or pos.shape[0] != n:
        raise ValueError(f"pos must have shape ({n},), got {tuple(pos.shape)}")
    if not pos.is_contiguous():
        raise ValueError("pos must be contiguous")
    if pos.dtype != torch.int32:
        raise ValueError(f"pos must be an int32 tensor, got {pos.dtype}")
    if freqs.ndim != 1 or freqs.shape[0] * 2 != d:
        raise ValueError(f"freqs must have shape ({d // 2},), got {tuple(freqs.shape)}")
    if not freqs.is_contiguous():
        raise ValueError("freqs must be contiguous")
    if freqs.dtype != torch.float32:
        raise ValueError(f"freqs must be a float32 tensor, got {freqs.dtype}")
    _dtype_code(x, "apply_rope")
    _require_cuda("apply_rope", x, pos, freqs)
    (_rope_op if _use_registered_op() else _rope_impl)(x, pos, freqs)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``(x * rsqrt(mean(x^2) + eps)) * w`` with fp32 accumulation
    (``cwm/fastgen/kernels/rmsnorm.py:64-119``); also stands in for the
    ``rms_norm(h, w, eps)`` calls of ``cwm/fastgen/forward.py:571,772,789``.

    ``x``: ``(N, D)`` contiguous; ``w``: ``(D,)`` contiguous, same dtype as ``x``.
    Returns a new tensor like ``x``.
    """
    if x.ndim != 2:
        raise ValueError(f"x must have 2 dimensions (N, D), got {x.ndim}")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    d = x.shape[1]
    if tuple(w.shape) != (d,):
        raise ValueError(f"w must have shape ({d},), got {tuple(w.shape)}")
    if not w.is_contiguous():
        raise ValueError("w must be contiguous")
    if w.dtype != x.dtype:
        raise ValueError(f"w must have the dtype of x ({x.dtype}), got {w.dtype}")
    _dtype_code(x, "rmsnorm")
    _require_cuda("rmsnorm", x, w)
    return (_rmsnorm_op if _use_registered_op() else _rmsnorm_impl)(x, w, float(eps))


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``h.add_(delta)`` followed by ``rmsnorm(h, w, eps)`` in one pass over the rows
    (the residual add and the next normalisation of ``cwm/fastgen/forward.py:769-772``
    and ``:786-789``).  ``h`` is updated in place, rounded to its dtype exactly as
    ``add_`` would; the normalised rows are returned as a new tensor."""
    if h.ndim != 2 or delta.shape != h.shape:
        raise ValueError("h and delta must be 2-D tensors of the same shape")
    if not h.is_contiguous() or not delta.is_contiguous():
        raise ValueError("h and delta must be contiguous")
    if delta.dtype != h.dtype or w.dtype != h.dtype:
        raise ValueError("h, delta and w must share a dtype")
    if tuple(w.shape) != (h.shape[1],) or not w.is_contiguous():
        raise ValueError(f"w must be a contiguous tensor of shape ({h.shape[1]},)")
    _dtype_code(h, "add_rmsnorm")
    _require_cuda("add_rmsnorm", h, delta, w)
    fn = _add_rmsnorm_op if _use_registered_op() else _add_rmsnorm_impl
    return fn(h, delta, w, float(eps))


def paged_memcpy(
    src: torch.Tensor,
    dst: torch.Tensor,
    page_tbl: torch.Tensor,
    dst_pos: torch.Tensor,
    dst_shard: tuple[int, int] | None,
    src_batch: torch.Tensor | None,
    batch_size: torch.Tensor | None,
    page_size: int,
) -> None:
    """Scatter the rows of ``src`` into the paged tensor ``dst``
    (``cwm/fastgen/kernels/paged_memcpy.py:90-228``).

    Row ``n`` is stored at ``dst[page_tbl[b, pos // page_size] * page_size +
    pos % page_size]`` with ``pos = dst_pos[n]`` and ``b = src_batch[n]`` (``n``
    when ``src_batch`` is None).  ``batch_size``, a 0-d int32/int64 device tensor,
    limits the copy to the first ``batch_size`` rows (for graph replays on
    padded batches).  ``dst_shard = (K, S)`` keeps only positions ``pos % S == K``
    and stores them at ``pos // S``.  ``dst`` may be a column slice of a wider
    tensor (unit stride in its last dimension).  As in the reference,
    ``src_batch`` and ``batch_size`` are mutually exclusive.
    """
    if src.ndim != 2 or dst.ndim != 2:
        raise ValueError(f"src and dst must be 2-D, got {src.ndim}-D and {dst.ndim}-D")
    if src.shape[1] != dst.shape[1]:
        raise ValueError("src and dst must agree on dimension 1")
    if src.dtype != dst.dtype:
        raise ValueError(f"src and dst must share a dtype, got {src.dtype} and {dst.dtype}")
    if not src.is_contiguous():
        raise ValueError("src must be contiguous")
    if dst.stride(1) != 1:
        raise ValueError("dst must have unit stride in its last dimension")
    n = src.shape[0]
    if page_tbl.ndim != 2:
        raise ValueError(f"page_tbl must be a 2-D int32 tensor, got shape {tuple(page_tbl.shape)}")
    if page_tbl.dtype != torch.int32:
        raise ValueError("page_tbl must be an int32 tensor")
    if page_tbl.shape[1] > 1 and page_tbl.stride(1) != 1:
        raise ValueError("page_tbl must have unit stride in its last dimension")
    if dst_pos.ndim != 1 or dst_pos.shape[0] != n:
        raise ValueError(f"dst_pos must have shape ({n},), got {tuple(dst_pos.shape)}")
    if dst_pos.dtype != torch.int32:
        raise ValueError(f"dst_pos must be an int32 tensor, got {dst_pos.dtype}")
    if not dst_pos.is_contiguous():
        raise ValueError("dst_pos must be contiguous")
    if src_batch is not None:
        if src_batch.ndim != 1 or src_batch.shape[0] != n:
            raise ValueError(f"src_batch must have shape ({n},), got {tuple(src_batch.shape)}")
        if src_batch.dtype != torch.int32:
            raise ValueError(f"src_batch must be an int32 tensor, got {src_batch.dtype}")
        if not src_batch.is_contiguous():
            raise ValueError("src_batch must be contiguous")
    if batch_size is not None:
        if batch_size.ndim != 0:
            raise ValueError(f"batch_size must be a 0-d tensor, got shape {tuple(batch_size.shape)}")
        if batch_size.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"batch_size must be int32 or int64, got {batch_size.dtype}")
        if src_batch is not None:
            raise ValueError("src_batch and batch_size cannot be given together")
    if dst_shard is not None:
        k, s = dst_shard
        if s < 1 or not 0 <= k < s:
            raise ValueError(f"dst_shard must be (K, S) with 0 <= K < S, got {dst_shard}")
    else:
        k, s = 0, 1
    if page_size <= 0:
        raise ValueError(f"page_size must be positive, got {page_size}")
    _require_cuda("paged_memcpy", src, dst, page_tbl, dst_pos, src_batch, batch_size)
    fn = _paged_memcpy_op if _use_registered_op() else _paged_memcpy_impl
    fn(src, dst, page_tbl, dst_pos, k, s, src_batch, batch_size, page_size)
