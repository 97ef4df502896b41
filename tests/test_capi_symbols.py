"""The C-ABI library builds (nvcc cross-compiles without a GPU), loads, and exports
every symbol that include/cwm_b200.h declares.  Only host-side argument checks are
exercised here: nothing is launched."""

from __future__ import annotations

import re
from pathlib import Path

from cwm_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols() -> list[str]:
    text = (ROOT / "include" / "cwm_b200.h").read_text()
    return re.findall(r"CWM_API\s+[\w\s\*]+?\b(cwm_\w+)\s*\(", text)


def test_header_symbols_are_exported_and_bound(lib):
    names = _declared_symbols()
    assert len(names) >= 11 and len(set(names)) == len(names)
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_every_entry_point_cites_the_reference_or_says_it_has_none():
    text = (ROOT / "include" / "cwm_b200.h").read_text()
    for name in ("cwm_rope", "cwm_rmsnorm", "cwm_paged_memcpy", "cwm_rope_kv_write",
                 "cwm_paged_attn_fwd"):
        decl = text.index(f" {name}(")
        comment = text.rfind("/*", 0, decl)
        assert "cwm/fastgen/" in text[comment:decl], name
    decl = text.index(" cwm_paged_attn_decode_noalloc(")
    assert "No counterpart in the reference" in text[text.rfind("/*", 0, decl):decl]


def test_version_and_error_strings(lib):
    assert lib.cwm_version() >= 1
    assert lib.cwm_strerror(_lib.CWM_OK) == b"ok"
    assert b"workspace" in lib.cwm_strerror(_lib.CWM_ERR_WORKSPACE)
    assert lib.cwm_paged_attn_workspace_bytes(64, 64, 48, 8, 128) > 2 * 34 * 32 * 4


def test_host_side_validation_without_a_gpu(lib):
    """Bad arguments are rejected before any CUDA call, so this runs on the CPU."""
    p = 0x1000  # never dereferenced
    # head_dim that is not built
    rc = lib.cwm_paged_attn_fwd(p, p, p, p, None, p, p, p, 1, 1, 8, 1, 64, 0, 256, 4, 128, 4, 1,
                                256, 1.0, -1, p, 1 << 30, None)
    assert rc == _lib.CWM_ERR_UNSUPPORTED and b"head_dim" in lib.cwm_last_error()
    # query heads not a multiple of KV heads
    rc = lib.cwm_paged_attn_fwd(p, p, p, p, None, p, p, p, 1, 1, 7, 2, 128, 0, 256, 4, 512, 4, 1,
                                256, 1.0, -1, p, 1 << 30, None)
    assert rc == _lib.CWM_ERR_INVALID
    # page size that the tiles cannot cover
    rc = lib.cwm_paged_attn_fwd(p, p, p, p, None, p, p, p, 1, 1, 8, 1, 128, 0, 48, 4, 256, 4, 1,
                                256, 1.0, -1, p, 1 << 30, None)
    assert rc == _lib.CWM_ERR_UNSUPPORTED and b"page_size" in lib.cwm_last_error()
    # null pointers
    assert lib.cwm_rope(None, p, p, 4, 2, 128, 0, None) == _lib.CWM_ERR_INVALID
    assert lib.cwm_rmsnorm(p, None, p, 4, 64, 1e-5, 0, None) == _lib.CWM_ERR_INVALID
    # odd head_dim for rope
    assert lib.cwm_rope(p, p, p, 4, 2, 127, 0, None) == _lib.CWM_ERR_INVALID
    # empty problems are fine and launch nothing
    assert lib.cwm_rope(None, None, None, 0, 2, 128, 0, None) == _lib.CWM_OK
    assert lib.cwm_paged_memcpy(None, None, None, None, None, None, 0, 0, 64, 2, 256, 1, 1, 64, 0,
                                0, 1, None) == _lib.CWM_OK
    # the scratch-free decode entry point states its batch limit
    rc = lib.cwm_paged_attn_decode_noalloc(p, p, p, p, None, p, p, p, 5000, 6, 1, 128, 0, 256, 4,
                                           256, 1, 256, 1.0, -1, None)
    assert rc == _lib.CWM_ERR_WORKSPACE
