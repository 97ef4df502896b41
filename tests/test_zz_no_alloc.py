"""The scratch-free decode entry point against the regular one.

``cwm_paged_attn_decode_noalloc`` serves embedders that cannot allocate device
memory when they call into the library (a plugin working inside buffers its host
application gave it, a serving loop with a frozen memory plan): its split-KV
scratch is a fixed array inside the library instead of a caller workspace.  The
test drives both entry points through the C ABI on the same inputs, twice in a
row with different batches, so that the second call runs over whatever the first
one left in the shared scratch.  Both entry points launch the same kernel on the
same grid, so their outputs must agree bit for bit; the oracle is consulted as
well.  This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""

from __future__ import annotations


import pytest
import torch

from oracle import ref_paged_gqa_attention
from tests.helpers import make_problem

pytestmark = pytest.mark.gpu

TOL = 2e-2  # the attention tests' bound (bf16 against the fp32 oracle)


def _call_noalloc(lib, pg, p, window_left, stream):
    k4, v4 = pg.kv_views()
    batch = pg.seqused_k.shape[0]
    out = torch.zeros_like(pg.q)
    lse = torch.zeros(p.hq, batch, device=pg.q.device)
    rc = lib.cwm_paged_attn_decode_noalloc(
        pg.q.data_ptr(), k4.data_ptr(), v4.data_ptr(), out.data_ptr(), lse.data_ptr(),
        pg.cu_seqlens_q.data_ptr(), pg.seqused_k.data_ptr(), pg.block_table.data_ptr(), batch,
        p.hq, p.hkv, p.d, 0, p.page_size, k4.shape[0], k4.stride(1), pg.block_table.stride(0),
        pg.block_table.shape[1] * p.page_size, p.d**-0.5, window_left, stream,
    )
    assert rc == 0, lib.cwm_last_error()
    return out, lse


def _call_workspace(lib, pg, p, window_left, stream):
    k4, v4 = pg.kv_views()
    batch = pg.seqused_k.shape[0]
    out = torch.zeros_like(pg.q)
    lse = torch.zeros(p.hq, batch, device=pg.q.device)
    need = lib.cwm_paged_attn_workspace_bytes(batch, batch, p.hq, p.hkv, p.d)
    ws = torch.zeros(need, dtype=torch.uint8, device=pg.q.device)
    rc = lib.cwm_paged_attn_fwd(
        pg.q.data_ptr(), k4.data_ptr(), v4.data_ptr(), out.data_ptr(), lse.data_ptr(),
        pg.cu_seqlens_q.data_ptr(), pg.seqused_k.data_ptr(), pg.block_table.data_ptr(), batch,
        batch, p.hq, p.hkv, p.d, 0, p.page_size, k4.shape[0], k4.stride(1),
        pg.block_table.stride(0), 1, pg.block_table.shape[1] * p.page_size, p.d**-0.5,
        window_left, ws.data_ptr(), ws.numel(), stream,
    )
    assert rc == 0, lib.cwm_last_error()
    return out, lse


def _compare(lib, p, window_left, device, with_oracle=True):
    from cwm_b200 import _lib

    with torch.cuda.device(device):
        pg = p.to(device)
        stream = torch.cuda.current_stream().cuda_stream
        out_ws, lse_ws = _call_workspace(lib, pg, p, window_left, stream)
        out_na, lse_na = _call_noalloc(lib, pg, p, window_left, stream)
        torch.cuda.synchronize()
        assert _lib.device_status(stream) == 0
    assert out_ws.abs().sum() > 0
    # same kernel, same grid, same merge order: bit for bit
    assert torch.equal(out_ws.view(torch.int16), out_na.view(torch.int16))
    assert torch.equal(lse_ws.view(torch.int32), lse_na.view(torch.int32))
    if with_oracle:
        k4, v4 = p.kv_views()
        want, _ = ref_paged_gqa_attention(p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table,
                                       p.d**-0.5, window_left)
        assert (out_na.cpu().float() - want).abs().max().item() <= TOL


def test_noalloc_decode_matches_workspace_decode_twice(lib):
    # first call: many long sequences, so that segments span CTAs and partials are used
    first = make_problem([1] * 24, [900 + 611 * i for i in range(24)], seed=101)
    # second call: fewer, shorter sequences and a sliding window, over the used scratch
    second = make_problem([1] * 5, [70, 0, 2000, 513, 256], hq=12, hkv=2, seed=102)
    for p, window_left in ((first, -1), (second, 255)):
        _compare(lib, p, window_left, "cuda:0")


def test_noalloc_decode_at_its_largest_batch(lib):
    """1024 sequences is the most the entry point accepts (and where the kernel's
    scheduler uses the most shared memory); short contexts keep the case small."""
    kv = [1 + (37 * i) % 700 for i in range(1024)]
    p = make_problem([1] * 1024, kv, hq=12, hkv=2, seed=103)
    _compare(lib, p, -1, "cuda:0", with_oracle=False)
    # oracle on a sample of the sequences
    pg = p.to("cuda:0")
    out, _ = _call_noalloc(lib, pg, p, -1, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    k4, v4 = p.kv_views()
    for b in (0, 1, 511, 1023):
        want, _ = ref_paged_gqa_attention(
            p.q[b : b + 1], k4, v4, torch.tensor([0, 1], dtype=torch.int32),
            p.seqused_k[b : b + 1], p.block_table[b : b + 1], p.d**-0.5, -1)
        assert (out[b : b + 1].cpu().float() - want).abs().max().item() <= TOL


def test_noalloc_decode_allocates_no_device_memory(lib):
    """After one warm-up call (the CUDA runtime loads kernels lazily), a second call
    leaves the device's free memory exactly where it was."""
    p = make_problem([1] * 8, [300 * (i + 1) for i in range(8)], hq=12, hkv=2, seed=104)
    pg = p.to("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    k4, v4 = pg.kv_views()
    batch = 8
    out = torch.zeros_like(pg.q)

    def call():
        rc = lib.cwm_paged_attn_decode_noalloc(
            pg.q.data_ptr(), k4.data_ptr(), v4.data_ptr(), out.data_ptr(), None,
            pg.cu_seqlens_q.data_ptr(), pg.seqused_k.data_ptr(), pg.block_table.data_ptr(),
            batch, p.hq, p.hkv, p.d, 0, p.page_size, k4.shape[0], k4.stride(1),
            pg.block_table.stride(0), pg.block_table.shape[1] * p.page_size, p.d**-0.5, -1,
            stream,
        )
        assert rc == 0, lib.cwm_last_error()
        torch.cuda.synchronize()

    call()
    free_before, _ = torch.cuda.mem_get_info(0)
    reserved_before = torch.cuda.memory_reserved(0)
    call()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before
    assert torch.cuda.memory_reserved(0) == reserved_before


def test_noalloc_decode_on_a_second_device(lib):
    """The scratch address is looked up once per device: a second GPU in the same
    process must get its own (plain local memory, no peer access involved)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    p = make_problem([1] * 6, [1500, 64, 4000, 257, 999, 3], hq=12, hkv=2, seed=105)
    _compare(lib, p, -1, "cuda:1")
    _compare(lib, p, 511, "cuda:0")


def test_noalloc_decode_rejects_oversized_batch(lib):
    from cwm_b200 import _lib

    t = torch.zeros(64, device="cuda:0")
    p = t.data_ptr()
    rc = lib.cwm_paged_attn_decode_noalloc(
        p, p, p, p, None, p, p, p, 1025, 6, 1, 128, 0, 256, 4, 256, 1, 256, 1.0, -1,
        torch.cuda.current_stream().cuda_stream,
    )
    assert rc == _lib.CWM_ERR_WORKSPACE
    assert b"1024" in lib.cwm_last_error()
