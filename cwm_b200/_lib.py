"""ctypes binding of ``libcwm_b200.so`` (the C ABI declared in ``include/cwm_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  The library is looked up next to this file; ``cwm_b200.build.build()``
produces it.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcwm_b200.so"

CWM_OK = 0
CWM_ERR_INVALID = 1
CWM_ERR_UNSUPPORTED = 2
CWM_ERR_CUDA = 3
CWM_ERR_WORKSPACE = 4

CWM_BF16, CWM_F16, CWM_F32 = 0, 1, 2

# name -> (restype, argtypes); must list every symbol of include/cwm_b200.h
SIGNATURES: dict[str, tuple] = {
    "cwm_version": (c_int, []),
    "cwm_strerror": (c_char_p, [c_int]),
    "cwm_last_error": (c_char_p, []),
    "cwm_device_status": (c_int, [ctypes.POINTER(c_int32), c_void_p]),
    "cwm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "cwm_rmsnorm": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_int, c_void_p],
    ),
    "cwm_add_rmsnorm": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_int, c_void_p],
    ),
    "cwm_paged_memcpy": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
         c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p],
    ),
    "cwm_rope_kv_write": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_int64,
         c_int64, c_int64, c_int64, c_void_p],
    ),
    "cwm_qkv_rope_kv_write": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64,
         c_int64, c_void_p],
    ),
    "cwm_block_copy": (
        c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p],
    ),
    "cwm_allreduce": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
    ),  # in, scratch table, result table, flag table, epoch, n, dtype, rank, world, stream
    "cwm_allreduce_add_rmsnorm": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
         c_float, c_int, c_int, c_int, c_void_p],
    ),  # in, h, w, scratch table, result table, flag table, epoch, rows, d, eps, dtype, rank, world, stream
    "cwm_allreduce_flag_ints": (c_int, []),
    "cwm_peer_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "cwm_peer_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "cwm_peer_close": (c_int, [c_void_p]),
    "cwm_peer_free": (c_int, [c_void_p]),
    "cwm_allreduce_ctas": (c_int, [c_int64, c_int]),
    "cwm_silu_mul": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "cwm_paged_attn_workspace_bytes": (c_size_t, [c_int, c_int64, c_int, c_int, c_int]),
    "cwm_test_hooks": (c_int, [ctypes.c_longlong, c_int]),
    "cwm_sample": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
         c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "cwm_paged_attn_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int,
         c_float, c_int, c_void_p, c_size_t, c_void_p],
    ),
    "cwm_paged_attn_decode_noalloc": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
         c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_float, c_int,
         c_void_p],
    ),
}

_lib: ctypes.CDLL | None = None


class CwmError(RuntimeError):
    """A call into libcwm_b200 failed for a reason other than a bad argument."""


def load() -> ctypes.CDLL:
    """Load the library once and declare the argument types of every symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise CwmError(
            f"{LIB_PATH} is missing: build it with `python -m cwm_b200.build` "
            "(there is no non-CUDA fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    """Turn a status code into the exception the reference would raise.

    Argument errors become ``ValueError`` (the reference validates before launch
    and raises ``ValueError``); everything else becomes ``CwmError``.
    """
    if code == CWM_OK:
        return
    lib = load()
    msg = lib.cwm_last_error().decode() or lib.cwm_strerror(code).decode()
    if code in (CWM_ERR_INVALID, CWM_ERR_UNSUPPORTED, CWM_ERR_WORKSPACE):
        raise ValueError(f"{what}: {msg}")
    raise CwmError(f"{what}: {msg}")


# callables run when the status word comes back non-zero (state to re-initialise)
on_bad_status: list = []


def device_status(stream_ptr: int = 0) -> int:
    """Read and clear the device status word (synchronises the stream).  A non-zero
    word means that the output of an earlier call is not valid; the registered
    clean-ups (``on_bad_status``) run before it is returned."""
    out = c_int32(0)
    check(load().cwm_device_status(ctypes.byref(out), stream_ptr), "cwm_device_status")
    if out.value != 0:
        for fn in on_bad_status:
            fn()
    return int(out.value)
