"""The scratch-free decode entry point against the regular one.

``cwm_paged_attn_decode_noalloc`` serves embedders that cannot allocate device
memory when they call into the library (a plugin working inside buffers its host
application gave it, a serving loop with a frozen memory plan): its split-KV
scratch is a fixed array inside the library instead of a caller workspace.  The
test drives both entry points through the C ABI on the same inputs, twice in a
row with different batches, so that the second call runs over whatever the first
one left in the shared scratch.  This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""

from __future__ import annotations


import pytest
import torch

from tests.helpers import make_problem

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = 2e-2  # the attention tests' bound (bf16 against the fp32 oracle)


def _call_both(lib, p, window_left):
    pg = p.to(DEV)
    k4, v4 = pg.kv_views()
    batch = pg.seqused_k.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    common = (
        pg.q.data_ptr(), k4.data_ptr(), v4.data_ptr(),
    )
    meta = (pg.cu_seqlens_q.data_ptr(), pg.seqused_k.data_ptr(), pg.block_table.data_ptr())
    max_k = pg.block_table.shape[1] * p.page_size
    scale = p.d**-0.5

    out_ws = torch.zeros_like(pg.q)
    lse_ws = torch.zeros(p.hq, batch, device=DEV)
    need = lib.cwm_paged_attn_workspace_bytes(batch, batch, p.hq, p.hkv, p.d)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    rc = lib.cwm_paged_attn_fwd(
        *common, out_ws.data_ptr(), lse_ws.data_ptr(), *meta, batch, batch, p.hq, p.hkv, p.d, 0,
        p.page_size, k4.shape[0], k4.stride(1), pg.block_table.stride(0), 1, max_k, scale,
        window_left, ws.data_ptr(), ws.numel(), stream,
    )
    assert rc == 0, lib.cwm_last_error()

    out_na = torch.zeros_like(pg.q)
    lse_na = torch.zeros(p.hq, batch, device=DEV)
    rc = lib.cwm_paged_attn_decode_noalloc(
        *common, out_na.data_ptr(), lse_na.data_ptr(), *meta, batch, p.hq, p.hkv, p.d, 0,
        p.page_size, k4.shape[0], k4.stride(1), pg.block_table.stride(0), max_k, scale,
        window_left, stream,
    )
    assert rc == 0, lib.cwm_last_error()
    torch.cuda.synchronize()
    return out_ws.cpu().float(), out_na.cpu().float(), lse_ws.cpu(), lse_na.cpu()


def test_noalloc_decode_matches_workspace_decode_twice(lib):
    # first call: many long sequences, so that segments span CTAs and partials are used
    first = make_problem([1] * 24, [900 + 611 * i for i in range(24)], seed=101)
    # second call: fewer, shorter sequences and a sliding window, over the used scratch
    second = make_problem([1] * 5, [70, 0, 2000, 513, 256], hq=12, hkv=2, seed=102)
    for p, window_left in ((first, -1), (second, 255)):
        out_ws, out_na, lse_ws, lse_na = _call_both(lib, p, window_left)
        assert out_ws.abs().sum() > 0
        assert (out_ws - out_na).abs().max().item() <= TOL
        finite = torch.isfinite(lse_ws)
        assert torch.equal(finite, torch.isfinite(lse_na))
        assert (lse_ws[finite] - lse_na[finite]).abs().max().item() <= TOL


def test_noalloc_decode_rejects_oversized_batch(lib):
    from cwm_b200 import _lib

    t = torch.zeros(64, device=DEV)
    p = t.data_ptr()
    rc = lib.cwm_paged_attn_decode_noalloc(
        p, p, p, p, None, p, p, p, 1025, 6, 1, 128, 0, 256, 4, 256, 1, 256, 1.0, -1,
        torch.cuda.current_stream().cuda_stream,
    )
    assert rc == _lib.CWM_ERR_WORKSPACE
    assert b"1024" in lib.cwm_last_error()
