"""Properties of the attention restatement that hold whatever the values are
(hypothesis-driven, CPU).  The attention oracle has no reference vectors to pin it,
so it is held to the invariants of the operation it restates instead."""

from __future__ import annotations

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import ref_paged_gqa_attention
from tests.helpers import make_problem


def _run(p, window_left, q=None, cache=None, table=None, seqk=None, cu=None):
    k4, v4 = p.kv_views(cache)
    return ref_paged_gqa_attention(
        p.q if q is None else q, k4, v4, p.cu_seqlens_q if cu is None else cu,
        p.seqused_k if seqk is None else seqk, p.block_table if table is None else table,
        p.d**-0.5, window_left)[0]


problems = st.builds(
    lambda seed, lens, page: (seed, lens, page),
    st.integers(0, 10_000),
    st.lists(st.tuples(st.integers(1, 9), st.integers(0, 40)), min_size=1, max_size=4),
    st.sampled_from([4, 8, 16]),
)


def _build(spec):
    seed, lens, page = spec
    q_lens = [t for t, _ in lens]
    kv = [t + n0 for t, n0 in lens]
    return make_problem(q_lens, kv, hq=4, hkv=2, d=8, page_size=page, seed=seed,
                        dtype=torch.float32)


@settings(max_examples=25, deadline=None)
@given(problems, st.integers(0, 30))
def test_page_placement_does_not_matter(spec, perm_seed):
    p = _build(spec)
    n_pages = p.cache.shape[0] // p.page_size
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(perm_seed))
    moved = torch.empty_like(p.cache)
    moved.view(n_pages, p.page_size, -1)[perm] = p.cache.view(n_pages, p.page_size, -1)
    table = perm[p.block_table.long()].to(torch.int32)
    assert torch.equal(_run(p, -1), _run(p, -1, cache=moved, table=table))


@settings(max_examples=25, deadline=None)
@given(problems)
def test_window_covering_the_context_is_global(spec):
    p = _build(spec)
    longest = int(p.seqused_k.max())
    assert torch.equal(_run(p, -1), _run(p, longest))
    assert torch.equal(_run(p, -1), _run(p, longest + 1000))


@settings(max_examples=25, deadline=None)
@given(problems, st.integers(0, 12))
def test_window_equals_attention_over_truncated_history(spec, window_left):
    """A query with window_left = w sees exactly what a global query would see if the
    keys older than w positions did not exist: check on single-query sequences by
    zero-weighting through an explicit softmax."""
    p = _build(spec)
    out = _run(p, window_left)
    k4, v4 = p.kv_views()
    cu = p.cu_seqlens_q.tolist()
    for b in range(len(cu) - 1):
        t, n = cu[b + 1] - cu[b], int(p.seqused_k[b])
        j = t - 1  # last query of the sequence, at position n - 1
        lo = max(0, n - 1 - window_left)
        keys = range(lo, n)
        rows = [(int(p.block_table[b, kk // p.page_size]), kk % p.page_size) for kk in keys]
        for h in range(p.hq):
            kh = h // (p.hq // p.hkv)
            kk = torch.stack([k4[pg, o, kh] for pg, o in rows])
            vv = torch.stack([v4[pg, o, kh] for pg, o in rows])
            w = torch.softmax((kk @ p.q[cu[b] + j, h]) * p.d**-0.5, dim=0)
            assert torch.allclose(out[cu[b] + j, h], w @ vv, atol=1e-5)


@settings(max_examples=25, deadline=None)
@given(problems)
def test_output_is_linear_in_v_and_invariant_to_unread_memory(spec):
    p = _build(spec)
    w = p.hkv * p.d
    base = _run(p, 3)
    doubled = p.cache.clone()
    doubled[:, w:] *= 2.0
    assert torch.allclose(_run(p, 3, cache=doubled), 2.0 * base, atol=1e-5)
    # rows beyond a sequence's length and pages outside its table are never read
    poisoned = p.cache.clone()
    used = torch.zeros(p.cache.shape[0], dtype=torch.bool)
    for b in range(p.seqused_k.shape[0]):
        n = int(p.seqused_k[b])
        for pos in range(n):
            used[int(p.block_table[b, pos // p.page_size]) * p.page_size + pos % p.page_size] = True
    poisoned[~used] = float("nan")
    assert torch.equal(_run(p, 3, cache=poisoned), base)


@settings(max_examples=25, deadline=None)
@given(problems)
def test_chunked_queries_equal_one_call(spec):
    """Feeding a sequence's new tokens in two calls (the second with the longer key
    count) gives the rows of the single call: what chunked prefill relies on."""
    p = _build(spec)
    whole = _run(p, 5)
    cu = p.cu_seqlens_q.tolist()
    for b in range(len(cu) - 1):
        t, n = cu[b + 1] - cu[b], int(p.seqused_k[b])
        if t < 2:
            continue
        cut = t // 2
        for q0, q1, keys in ((0, cut, n - (t - cut)), (cut, t, n)):
            part = ref_paged_gqa_attention(
                p.q[cu[b] + q0 : cu[b] + q1], *p.kv_views(),
                torch.tensor([0, q1 - q0], dtype=torch.int32),
                torch.tensor([keys], dtype=torch.int32), p.block_table[b : b + 1], p.d**-0.5, 5)[0]
            assert torch.allclose(part, whole[cu[b] + q0 : cu[b] + q1], atol=1e-6)
