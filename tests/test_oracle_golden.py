"""The CPU oracle against the golden vectors made by the reference's own Triton
kernels (run under the Triton interpreter; see tests/golden/make_golden.py), and
self-consistency checks of the attention restatement, which has no reference
vectors (parity unpinned)."""

from __future__ import annotations

import numpy as np
import torch

from oracle import (
    ref_gqa_attention_layer,
    ref_paged_gqa_attention,
    ref_paged_memcpy,
    ref_rmsnorm,
    ref_rope,
    ref_rope_freqs,
)
from tests.helpers import make_problem


def test_rope_matches_reference_kernel(golden):
    for name in ("small", "grouped"):
        x = torch.from_numpy(golden[f"rope_{name}_x"].copy())
        pos = torch.from_numpy(golden[f"rope_{name}_pos"])
        freqs = torch.from_numpy(golden[f"rope_{name}_freqs"])
        want = torch.from_numpy(golden[f"rope_{name}_out"])
        ref_rope(x, pos, freqs)
        # fp32 in and out; sin/cos implementations may differ in the last ulp
        assert torch.allclose(x, want, rtol=0, atol=2e-6), (x - want).abs().max()


def test_rope_freqs_expression(golden):
    f = ref_rope_freqs(128, 1e6)
    assert np.array_equal(f.numpy(), golden["rope_small_freqs"])
    scaled = ref_rope_freqs(
        128, 5e5,
        dict(low_freq_factor=1, high_freq_factor=4, old_context_len=8192, scale_factor=8),
    )
    plain = ref_rope_freqs(128, 5e5)
    assert scaled[0] == plain[0] and torch.isclose(scaled[-1], plain[-1] / 8)


def test_rmsnorm_matches_reference_kernel(golden):
    for name in ("cwm", "odd"):
        x = torch.from_numpy(golden[f"rms_{name}_x"])
        w = torch.from_numpy(golden[f"rms_{name}_w"])
        eps = float(golden[f"rms_{name}_eps"])
        want = torch.from_numpy(golden[f"rms_{name}_out"])
        got = ref_rmsnorm(x, w, eps)
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), (got - want).abs().max()


def _memcpy_case(golden, name):
    meta = golden[f"mc_{name}_meta"]
    page, n_pages, b, bs, k, s, kv_view, is16 = (int(v) for v in meta)
    src = torch.from_numpy(golden[f"mc_{name}_src"].copy())
    full_want = torch.from_numpy(golden[f"mc_{name}_full"].copy())
    if is16:
        src = src.view(torch.bfloat16)
        full_want = full_want.view(torch.bfloat16)
    tbl = torch.from_numpy(golden[f"mc_{name}_tbl"])
    pos = torch.from_numpy(golden[f"mc_{name}_pos"])
    key = f"mc_{name}_src_batch"
    src_batch = torch.from_numpy(golden[key]) if key in golden.files else None
    return dict(
        src=src, full_want=full_want, tbl=tbl, pos=pos, src_batch=src_batch, page=page,
        batch_size=None if bs < 0 else bs, shard=(k, s) if s > 1 else None, kv_view=bool(kv_view),
    )


MEMCPY_CASES = ("prefill_bf16", "decode_bf16", "shard_f32", "wide_f32")


def test_paged_memcpy_matches_reference_kernel(golden):
    for name in MEMCPY_CASES:
        c = _memcpy_case(golden, name)
        full = torch.zeros_like(c["full_want"])
        e = c["src"].shape[1]
        dst = full[:, e:] if c["kv_view"] else full
        ref_paged_memcpy(
            c["src"], dst, c["tbl"], c["pos"], c["shard"], c["src_batch"], c["batch_size"],
            c["page"],
        )
        assert torch.equal(full.view(torch.uint8), c["full_want"].view(torch.uint8)), name


def _naive_attention(p, window_left):
    """Independent scalar-loop restatement for tiny cases."""
    q = p.q.float()
    k4, v4 = p.kv_views()
    group = p.hq // p.hkv
    out = torch.zeros_like(q)
    cu = p.cu_seqlens_q.tolist()
    for b in range(len(cu) - 1):
        t, n = cu[b + 1] - cu[b], int(p.seqused_k[b])
        for j in range(t):
            pos = n - t + j
            lo = 0 if window_left < 0 else max(0, pos - window_left)
            keys = list(range(lo, pos + 1)) if pos >= 0 else []
            if not keys:
                continue
            rows = [(int(p.block_table[b, kk // p.page_size]), kk % p.page_size) for kk in keys]
            for h in range(p.hq):
                kh = h // group
                kk = torch.stack([k4[pg, o, kh].float() for pg, o in rows])
                vv = torch.stack([v4[pg, o, kh].float() for pg, o in rows])
                s = (kk @ q[cu[b] + j, h]) * p.d**-0.5
                w = torch.softmax(s, dim=0)
                out[cu[b] + j, h] = w @ vv
    return out


def test_attention_oracle_against_scalar_loops():
    p = make_problem([1, 5, 1, 3], [9, 12, 1, 3], hq=4, hkv=2, d=16, page_size=4, seed=3,
                     dtype=torch.float32)
    k4, v4 = p.kv_views()
    for wl in (-1, 0, 2, 5):
        got, lse = ref_paged_gqa_attention(
            p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table, p.d**-0.5, wl
        )
        want = _naive_attention(p, wl)
        assert torch.allclose(got, want, atol=1e-5), (wl, (got - want).abs().max())
        assert torch.isfinite(lse).all()


def test_attention_oracle_against_sdpa():
    """One sequence, no paging subtleties: compare with torch's dense attention."""
    p = make_problem([7], [19], hq=6, hkv=2, d=32, page_size=8, seed=5, dtype=torch.float32)
    k4, v4 = p.kv_views()
    got, _ = ref_paged_gqa_attention(
        p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table, p.d**-0.5, -1
    )
    pages = p.block_table[0, :3].long()
    k = k4[pages].reshape(-1, 2, 32)[:19].repeat_interleave(3, dim=1)
    v = v4[pages].reshape(-1, 2, 32)[:19].repeat_interleave(3, dim=1)
    mask = torch.ones(7, 19, dtype=torch.bool).tril(diagonal=19 - 7)
    want = torch.nn.functional.scaled_dot_product_attention(
        p.q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), attn_mask=mask
    ).transpose(0, 1)
    assert torch.allclose(got, want, atol=1e-5)


def test_attention_oracle_empty_and_windowed_rows():
    p = make_problem([1, 1, 2], [0, 1, 1], hq=2, hkv=1, d=8, page_size=4, seed=1,
                     dtype=torch.float32)
    k4, v4 = p.kv_views()
    out, lse = ref_paged_gqa_attention(
        p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table, 1.0, -1
    )
    assert torch.equal(out[0], torch.zeros_like(out[0])) and torch.isinf(lse[:, 0]).all()
    # one key: output is that value row, whatever the score
    v_row = v4[int(p.block_table[1, 0]), 0, 0].float()
    assert torch.allclose(out[1, 0], v_row) and torch.allclose(out[1, 1], v_row)
    # sequence 2 has 2 queries and 1 key: query 0 sits at position -1 and sees nothing
    assert torch.equal(out[2], torch.zeros_like(out[2]))
    assert torch.isfinite(out[3]).all() and out[3].abs().sum() > 0


def test_layer_oracle_writes_before_attending():
    """The new token must be visible to its own query (forward.py:621-655)."""
    torch.manual_seed(0)
    hq, hkv, d, page = 4, 2, 16, 4
    cache = torch.zeros(3 * page, hkv * 2 * d)
    table = torch.tensor([[2, 0]], dtype=torch.int32)
    freqs = ref_rope_freqs(d, 1e4)
    xq, xk, xv = torch.randn(1, hq, d), torch.randn(1, hkv, d), torch.randn(1, hkv, d)
    out = ref_gqa_attention_layer(
        xq, xk, xv.clone(), cache, torch.tensor([0], dtype=torch.int32), None, None, freqs,
        torch.tensor([0, 1], dtype=torch.int32), torch.tensor([1], dtype=torch.int32), table,
        page, -1,
    )
    # a single key: the output equals the value just written, for every head of the group
    assert torch.allclose(out[0, 0], xv[0, 0]) and torch.allclose(out[0, 3], xv[0, 1])
    assert torch.equal(cache[2 * page, hkv * d :], xv.flatten())
    assert torch.equal(cache[2 * page, : hkv * d], xk.flatten())  # xk was rotated in place
