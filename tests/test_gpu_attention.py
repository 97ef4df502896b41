"""GPU parity of paged GQA attention (decode split-KV kernel and prefill kernel)
through the C ABI against the CPU fp32 oracle on the same seeded inputs.

Tolerance of the path: max-abs 2e-2 for bf16 inputs against the fp32 oracle
evaluated on the same bf16-rounded values."""

from __future__ import annotations

import math

import pytest
import torch

from oracle import ref_paged_gqa_attention
from tests.helpers import make_problem

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = 2e-2


@pytest.fixture(scope="module")
def ops(lib):
    import cwm_b200

    return cwm_b200


def _status():
    from cwm_b200 import _lib

    return _lib.device_status(torch.cuda.current_stream().cuda_stream)


def _run(ops, p, window_left, max_k=None):
    pg = p.to(DEV)
    k4, v4 = pg.kv_views()
    q_lens = (p.cu_seqlens_q[1:] - p.cu_seqlens_q[:-1]).tolist()
    out, lse = ops.mha_fwd(
        query=pg.q, key=k4, value=v4, cu_seqlens_q=pg.cu_seqlens_q, cu_seqlens_k=None,
        seqused_k=pg.seqused_k, leftpad_k=None, max_seqlen_q=max(q_lens + [0]),
        max_seqlen_k=max_k if max_k is not None else p.block_table.shape[1] * p.page_size,
        p=0, block_table=pg.block_table, softmax_scale=p.d**-0.5, is_causal=True,
        window_left=window_left, window_right=-1,
    )
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu()


def _check(ops, p, window_left, **kw):
    got, lse = _run(ops, p, window_left, **kw)
    k4, v4 = p.kv_views()
    want, want_lse = ref_paged_gqa_attention(
        p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table, p.d**-0.5, window_left
    )
    err = (got.float() - want).abs().max().item()
    assert err <= TOL, f"max-abs {err}"
    finite = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(lse), finite)
    assert (lse[finite] - want_lse[finite]).abs().max().item() <= 1e-2 if finite.any() else True
    assert _status() == 0
    return got


# ---------------------------------------------------------------------- decode
def test_decode_config1_shapes(ops):
    """Batch 4, 48/8 heads, contexts in [512, 2048], page 256, random placement."""
    g = torch.Generator().manual_seed(1001)
    ctx = torch.randint(512, 2049, (4,), generator=g).tolist()
    p = make_problem([1] * 4, ctx, seed=1001)
    _check(ops, p, -1)
    _check(ops, p, 8191)


@pytest.mark.parametrize("ctx", [1, 2, 15, 16, 17, 63, 64, 65, 255, 256, 257, 511, 513])
def test_decode_page_and_tile_boundaries(ops, ctx):
    p = make_problem([1, 1], [ctx, max(1, ctx - 1)], seed=ctx)
    _check(ops, p, -1)


@pytest.mark.parametrize("window", [0, 1, 63, 64, 100, 255, 256, 8191])
def test_decode_sliding_window(ops, window):
    p = make_problem([1, 1, 1], [700, 8200, 257], hq=12, hkv=2, seed=window)
    _check(ops, p, window)


@pytest.mark.parametrize("ctx", [8191, 8192, 8193, 20000])
def test_decode_window_8192_boundaries(ops, ctx):
    p = make_problem([1], [ctx], hq=6, hkv=1, seed=ctx)
    _check(ops, p, 8191)
    _check(ops, p, -1)


@pytest.mark.parametrize("hq,hkv", [(48, 8), (24, 4), (12, 2), (6, 1), (8, 8), (16, 2), (3, 1)])
def test_decode_head_groupings(ops, hq, hkv):
    p = make_problem([1] * 3, [300, 1000, 77], hq=hq, hkv=hkv, seed=hq * 10 + hkv)
    _check(ops, p, -1)


def test_decode_many_sequences_long_contexts(ops):
    """Enough work for several tiles per CTA, so segments end inside CTAs and
    others span CTA boundaries (direct writes and combined partials both occur)."""
    g = torch.Generator().manual_seed(2)
    ctx = [int(math.exp(v)) for v in torch.empty(48).uniform_(math.log(600), math.log(9000), generator=g)]
    p = make_problem([1] * 48, ctx, seed=2)
    _check(ops, p, -1)
    _check(ops, p, 2047)


def test_decode_empty_and_padded_lanes(ops):
    """Lanes with no keys (graph padding) give zero rows and -inf lse."""
    p = make_problem([1] * 5, [0, 300, 0, 1, 0], hq=12, hkv=2, seed=7)
    got = _check(ops, p, -1)
    assert got[0].abs().sum() == 0 and got[2].abs().sum() == 0 and got[4].abs().sum() == 0


def test_decode_static_bound_larger_than_lengths(ops):
    """max_seqlen_k is only an upper bound in graph-captured decode."""
    p = make_problem([1] * 3, [100, 900, 300], hq=12, hkv=2, seed=8, table_cols=40)
    _check(ops, p, -1, max_k=40 * 256)


def test_decode_row_sliced_block_table_and_fp16(ops):
    p = make_problem([1] * 6, [100, 200, 300, 400, 500, 600], hq=12, hkv=2, seed=11,
                     dtype=torch.float16)
    pg = p.to(DEV)
    k4, v4 = pg.kv_views()
    sl = slice(2, 5)
    out, _ = ops.mha_fwd(pg.q[sl], k4, v4, torch.arange(4, dtype=torch.int32, device=DEV), None,
                         pg.seqused_k[sl].contiguous(), None, 1, 768, 0, pg.block_table[sl],
                         p.d**-0.5, True, -1, -1)
    want, _ = ref_paged_gqa_attention(p.q[sl], *p.kv_views(), torch.arange(4, dtype=torch.int32),
                                      p.seqused_k[sl], p.block_table[sl], p.d**-0.5, -1)
    assert (out.cpu().float() - want).abs().max().item() <= TOL


def test_decode_is_deterministic(ops):
    p = make_problem([1] * 16, [3000 + 517 * i for i in range(16)], seed=5)
    a, _ = _run(ops, p, -1)
    b, _ = _run(ops, p, -1)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_decode_flags_bad_block_id(ops):
    p = make_problem([1], [600], hq=6, hkv=1, seed=3)
    p.block_table[0, 1] = 10_000
    _status()
    _run(ops, p, -1)
    assert _status() & 1


# --------------------------------------------------------------------- prefill
@pytest.mark.parametrize("t,n0", [(2, 0), (17, 0), (128, 0), (129, 5), (300, 0), (300, 700),
                                  (64, 192), (1, 1), (255, 1)])
def test_prefill_single_sequence(ops, t, n0):
    p = make_problem([t], [n0 + t], hq=12, hkv=2, seed=t + n0)
    _check(ops, p, -1)


@pytest.mark.parametrize("window", [0, 5, 63, 64, 127, 128, 300])
def test_prefill_sliding_window(ops, window):
    p = make_problem([200, 333], [200 + 100, 333 + 420], hq=6, hkv=1, seed=window)
    _check(ops, p, window)


def test_prefill_chunked_with_cached_prefix_full_heads(ops):
    """Several sequences, ragged chunk lengths, cached prefixes, 48/8 heads."""
    p = make_problem([256, 31, 500, 130], [256 + 1000, 31, 500 + 77, 130 + 2048], seed=21)
    _check(ops, p, -1)
    _check(ops, p, 511)


def test_prefill_window_8192(ops):
    p = make_problem([384], [384 + 9000], hq=6, hkv=1, seed=22)
    _check(ops, p, 8191)


def test_prefill_more_queries_than_keys(ops):
    """Queries that sit before position 0 see nothing and give zero rows."""
    p = make_problem([10], [4], hq=6, hkv=1, seed=23)
    got = _check(ops, p, -1)
    assert got[:6].abs().sum() == 0


def test_mixed_prefill_and_decode_one_call(ops):
    """One varlen launch with prefill chunks and single-token decodes."""
    q_lens = [1, 200, 1, 1, 130, 1]
    kv = [900, 200, 1, 5000, 130 + 300, 0]
    p = make_problem(q_lens, kv, seed=31)
    _check(ops, p, -1)
    _check(ops, p, 1023)


def test_prefill_is_deterministic(ops):
    p = make_problem([300, 200], [1300, 200], hq=12, hkv=2, seed=33)
    a, _ = _run(ops, p, 255)
    b, _ = _run(ops, p, 255)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


# ------------------------------------------------------------------ validation
def test_mha_fwd_rejects_what_is_not_built(ops):
    p = make_problem([1], [10], hq=6, hkv=1, seed=0).to(DEV)
    k4, v4 = p.kv_views()
    args = dict(query=p.q, key=k4, value=v4, cu_seqlens_q=p.cu_seqlens_q, cu_seqlens_k=None,
                seqused_k=p.seqused_k, leftpad_k=None, max_seqlen_q=1, max_seqlen_k=256, p=0,
                block_table=p.block_table, softmax_scale=1.0, is_causal=True, window_left=-1,
                window_right=-1)
    for bad in (dict(is_causal=False), dict(p=0.1), dict(cu_seqlens_k=p.cu_seqlens_q),
                dict(query=p.q.float()), dict(seqused_k=p.seqused_k.long()),
                dict(block_table=p.block_table.long()), dict(query=p.q[:, :, ::2]),
                dict(key=k4[:, :, :, ::2])):
        with pytest.raises(ValueError):
            ops.mha_fwd(**{**args, **bad})
    d64 = make_problem([1], [10], hq=2, hkv=1, d=64, seed=0).to(DEV)
    k4, v4 = d64.kv_views()
    with pytest.raises(ValueError):
        ops.mha_fwd(**{**args, "query": d64.q, "key": k4, "value": v4})


# ------------------------------------------------------------ KV-head sharding
@pytest.mark.parametrize("world", [2, 4, 8])
def test_head_sharded_runs_concatenate_to_the_unsharded_result(ops, world):
    """What each tensor-parallel rank computes on its own KV heads (local cache rows
    ``[K_local | V_local]``, local query heads) is the matching slice of the
    unsharded result.  The prefill kernel treats every (query block, head)
    independently, so its rows agree bit for bit; the decode kernel divides its
    tile list differently when the head count changes, so its rows agree within
    the tolerance of the path."""
    from cwm_b200.tp import shard_cache_rows, shard_heads

    q_lens = [1, 300, 1, 130]
    p = make_problem(q_lens, [2000, 300 + 900, 77, 130], seed=41)
    full, _ = _run(ops, p, 1023)
    decode_rows = torch.tensor([0, 301])
    prefill_rows = torch.tensor([r for r in range(sum(q_lens)) if r not in (0, 301)])
    parts = []
    for rank in range(world):
        sh = shard_heads(rank, world, p.hq, p.hkv)
        local = type(p)(
            p.q[:, sh.q_begin : sh.q_end].contiguous(), shard_cache_rows(p.cache, sh, p.hkv, p.d),
            p.cu_seqlens_q, p.seqused_k, p.block_table, p.page_size, sh.n_q, sh.n_kv, p.d,
        )
        out, _ = _run(ops, local, 1023)
        parts.append(out)
    cat = torch.cat(parts, dim=1)
    assert torch.equal(cat[prefill_rows].view(torch.int16), full[prefill_rows].view(torch.int16))
    assert (cat[decode_rows].float() - full[decode_rows].float()).abs().max().item() <= TOL
    assert _status() == 0


# ------------------------------------------------- shapes beyond the CWM defaults
@pytest.mark.parametrize("page_size", [64, 128, 512])
def test_other_page_sizes(ops, page_size):
    """Pages smaller than a 128-token prefill tile (two page lookups per tile) and
    larger than the default."""
    p = make_problem([1, 200, 1, 300], [700, 200 + 333, 65, 300], hq=12, hkv=2,
                     page_size=page_size, seed=page_size)
    _check(ops, p, -1)
    _check(ops, p, 100)


@pytest.mark.parametrize("hq,hkv", [(3, 1), (1, 1), (5, 5), (8, 1), (16, 4)])
def test_prefill_head_groupings(ops, hq, hkv):
    """Odd group sizes pair two consecutive 128-row blocks of one head in a CTA, even
    ones pair two heads; both with ragged lengths around the 128/256-row units."""
    p = make_problem([2, 128, 129, 256, 257, 500], [2, 128 + 40, 129, 256 + 300, 257, 500 + 77],
                     hq=hq, hkv=hkv, seed=hq * 7 + hkv)
    _check(ops, p, -1)
    _check(ops, p, 190)


def test_prefill_fp16(ops):
    p = make_problem([300, 140], [300 + 500, 140], hq=12, hkv=2, seed=51, dtype=torch.float16)
    _check(ops, p, -1)
    _check(ops, p, 255)


def test_large_batch_decode_and_prefill(ops):
    """More sequences than one scan step of the schedulers covers (batch > 32) and more
    decode segments than persistent CTAs."""
    g = torch.Generator().manual_seed(61)
    n = 400
    kv = torch.randint(1, 400, (n,), generator=g).tolist()
    q_lens = [1] * n
    for i in range(0, n, 50):
        q_lens[i] = min(kv[i], 70)
    p = make_problem(q_lens, kv, hq=6, hkv=1, seed=61)
    _check(ops, p, -1)


def test_randomized_problems(ops):
    """Seeded random batches: lengths, head groupings, windows, page sizes and the
    mix of decode and prefill sequences all vary."""
    g = torch.Generator().manual_seed(20250)

    def rnd(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=g))

    for case in range(12):
        hkv = [1, 2, 4][rnd(0, 2)]
        group = [1, 2, 3, 6, 8][rnd(0, 4)]
        page = [64, 128, 256][rnd(0, 2)]
        batch = rnd(1, 9)
        q_lens, kv = [], []
        for _ in range(batch):
            kind = rnd(0, 2)
            t = 1 if kind == 0 else rnd(2, 400)
            n0 = 0 if rnd(0, 3) == 0 else rnd(0, 1500)
            q_lens.append(t)
            kv.append(n0 + t if rnd(0, 9) else max(0, t - rnd(0, t)))  # sometimes fewer keys than queries
        window = [-1, 0, 37, 128, 700, 8191][rnd(0, 5)]
        p = make_problem(q_lens, kv, hq=hkv * group, hkv=hkv, page_size=page, seed=1000 + case)
        _check(ops, p, window)


def test_prefill_many_items_per_cluster(ops):
    """More work items than the persistent grid has clusters, of very different
    lengths, so that every cluster walks several items and its rings, score slots and
    barrier phases run on from one item to the next (odd and even tile counts, one-tile
    items, items whose queries see no key at all in between)."""
    g = torch.Generator().manual_seed(77)
    q_lens, kv = [], []
    for i in range(40):
        t = int(torch.randint(2, 300, (1,), generator=g))
        kind = i % 5
        if kind == 0:
            n = t  # no cached prefix
        elif kind == 1:
            n = t + int(torch.randint(1, 2500, (1,), generator=g))
        elif kind == 2:
            n = max(0, t - 130)  # the first queries sit before position 0
        elif kind == 3:
            n = 0  # no key at all: every work item of the sequence is empty
        else:
            n = t + 128 * int(torch.randint(0, 6, (1,), generator=g))
        q_lens.append(t)
        kv.append(n)
    for hq, hkv in ((12, 2), (3, 1)):
        p = make_problem(q_lens, kv, hq=hq, hkv=hkv, seed=770 + hq)
        _check(ops, p, -1)
        _check(ops, p, 300)


def test_prefill_long_item_lists_are_deterministic(ops):
    """Two runs over a long item list give the same bits (tile-to-group assignment and
    buffer reuse depend only on the list, not on timing)."""
    p = make_problem([700, 64, 1000, 129, 2, 513], [700 + 3000, 64, 1000 + 100, 129 + 900, 2, 513],
                     hq=12, hkv=2, seed=78)
    a, _ = _run(ops, p, 1023)
    b, _ = _run(ops, p, 1023)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    _check(ops, p, 1023)


def test_decode_never_uses_rows_beyond_the_context(ops):
    """Rows of the last page at or beyond ``seqused_k`` hold whatever the page held
    before; filled with NaN and Inf they must not change a bit of the decode output
    (P = 0 times NaN would otherwise poison the row through the P.V product)."""
    ctx = [70, 300, 1000, 513, 255, 64, 1]
    p = make_problem([1] * len(ctx), ctx, hq=12, hkv=2, seed=91)
    clean, _ = _run(ops, p, -1)
    clean_w, _ = _run(ops, p, 127)
    poisoned = make_problem([1] * len(ctx), ctx, hq=12, hkv=2, seed=91)
    rows = poisoned.cache.view(-1, p.page_size, poisoned.cache.shape[1])
    for b, n in enumerate(ctx):
        last = (n - 1) // p.page_size
        page = int(p.block_table[b, last])
        rows[page, n - last * p.page_size :] = float("nan")
        rows[page, n - last * p.page_size :: 2] = float("inf")
    got, _ = _run(ops, poisoned, -1)
    got_w, _ = _run(ops, poisoned, 127)
    assert torch.isfinite(got).all() and torch.isfinite(got_w).all()
    assert torch.equal(got.view(torch.int16), clean.view(torch.int16))
    assert torch.equal(got_w.view(torch.int16), clean_w.view(torch.int16))
    assert _status() == 0


def test_too_small_max_seqlen_q_is_reported(ops):
    """max_seqlen_q is a promise of the caller; one that understates it gets status
    bit 4 instead of silence."""
    p = make_problem([300, 40], [300, 500], hq=12, hkv=2, seed=92)
    pg = p.to(DEV)
    k4, v4 = pg.kv_views()
    ops.mha_fwd(pg.q, k4, v4, pg.cu_seqlens_q, None, pg.seqused_k, None, 128,
                p.block_table.shape[1] * p.page_size, 0, pg.block_table, p.d**-0.5, True, -1, -1)
    torch.cuda.synchronize()
    assert _status() & 4
    # one-query sequences although the bounds promised none: the decode kernel did not run
    p2 = make_problem([1, 3], [50, 60], hq=12, hkv=2, seed=93)
    pg2 = p2.to(DEV)
    k4, v4 = pg2.kv_views()
    cu = torch.tensor([0, 1, 4], dtype=torch.int32, device=DEV)
    q = torch.randn(4, 12, 128, device=DEV).to(torch.bfloat16)
    # total_q == batch * max_seqlen_q tells the library that every sequence has 2 queries
    ops.mha_fwd(q, k4, v4, cu, None, pg2.seqused_k, None, 2, p2.block_table.shape[1] * p2.page_size,
                0, pg2.block_table, p2.d**-0.5, True, -1, -1)
    torch.cuda.synchronize()
    assert _status() & 4
    good, _ = _run(ops, p, -1)  # the next correct call is unaffected
    assert _status() == 0 and torch.isfinite(good).all()
