"""A second opinion on the attention oracle's mask conventions.

The reference's attention arithmetic lives in a third-party FlashAttention-3
binding that is not available here, so the oracle's three conventions -- an
inclusive window of ``window_left + 1`` keys ending at the query itself, causal
alignment to the *end* of the key sequence when a cached prefix exists, and
contiguous grouping of query heads over KV heads -- cannot be pinned to the
reference.  The ``flash_attn`` package installed in this image is an independent
implementation of the same published FlashAttention varlen / paged-KV interface
(``causal=True``, ``window_size=(left, 0)``, ``block_table``).  Where its kernel
launches on this GPU it is run as a library call on the boundary cases of the
attention tests and compared with the oracle; if it cannot be imported or its
kernel has no image for this GPU, the test is skipped with that error.  It is a
cross-check of the oracle, not the reference and not part of the product path.
"""

from __future__ import annotations

import pytest
import torch

from oracle import ref_paged_gqa_attention
from tests.helpers import make_problem

pytestmark = pytest.mark.gpu

DEV = "cuda:0"

CASES = [
    # (q_lens, kv_lens, window_left)
    ([1, 1, 1], [700, 256, 257], -1),          # decode, page boundaries
    ([1, 1, 1], [700, 256, 257], 0),           # window of the query itself only
    ([1, 1], [700, 300], 1),
    ([1, 1, 1], [1000, 256, 600], 255),        # window ending one short of a page
    ([1, 1, 1], [1000, 256, 600], 256),
    ([1, 1], [9000, 8192], 8191),              # CWM's local layer
    ([200, 131], [300, 131], -1),              # prefill with and without cached prefix
    ([200, 131, 2], [300, 131, 515], 127),
    ([256, 64], [1024, 64], 255),
    ([64], [5000], 8191),
]


def _flash_attn():
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception as e:  # not importable in this environment
        pytest.skip(f"flash_attn cannot be imported: {e!r}")
    return flash_attn_varlen_func


@pytest.mark.parametrize("q_lens,kv_lens,window_left", CASES)
def test_oracle_agrees_with_flash_attn(q_lens, kv_lens, window_left):
    fa = _flash_attn()
    p = make_problem(q_lens, kv_lens, hq=12, hkv=2, seed=len(q_lens) * 1000 + kv_lens[0])
    pg = p.to(DEV)
    k4, v4 = pg.kv_views()
    # the library wants contiguous [pages, page, heads, dim] caches
    k4, v4 = k4.contiguous(), v4.contiguous()
    cu_k = torch.zeros(len(kv_lens) + 1, dtype=torch.int32)
    cu_k[1:] = torch.tensor(kv_lens).cumsum(0)
    try:
        got = fa(pg.q, k4, v4, pg.cu_seqlens_q, cu_k.to(DEV), max(q_lens), max(kv_lens),
                 softmax_scale=p.d**-0.5, causal=True,
                 window_size=(window_left, 0) if window_left >= 0 else (-1, -1),
                 block_table=pg.block_table)
        torch.cuda.synchronize()
    except RuntimeError as e:
        pytest.skip(f"flash_attn kernel did not launch on this GPU: {e}")
    ck4, cv4 = p.kv_views()
    want, _ = ref_paged_gqa_attention(p.q, ck4, cv4, p.cu_seqlens_q, p.seqused_k, p.block_table,
                                      p.d**-0.5, window_left)
    err = (got.cpu().float() - want).abs().max().item()
    assert err <= 2e-2, f"oracle and flash_attn disagree by {err}"
