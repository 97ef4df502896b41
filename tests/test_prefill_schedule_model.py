"""Model of the prefill kernel's work list and ring arithmetic
(cwm_b200/csrc/attn_prefill.cu): every cluster of the persistent grid walks the items
``cluster, cluster + n_clusters, ...`` of a list of (query block, head unit) pairs; a
KV tile gets a running number g over all items of a cluster, which alone decides the
softmax group (g % 2), the score slot and P buffer (g % 2), the K / V stage, the
"scores ready" and "product done" barriers (g % 4) and the "P ready" barrier (g % 4),
each with phase (g // ring) % 2.  This restates that arithmetic in Python and checks
its invariants on random batches: every (sequence, 128-row block, head) is covered once,
the tile range of an item covers every key a row may see, and with the kernel's
dependencies a barrier phase is never completed twice before its waiter has looked at
it.  It guards the rule, not the CUDA code (the GPU tests do that)."""

from __future__ import annotations

import random

BM = BN = 128


def blocks_of(q_lens, pair_heads):
    unit_rows = BM if pair_heads else 2 * BM
    prefix = [0]
    for t in q_lens:
        prefix.append(prefix[-1] + ((t + unit_rows - 1) // unit_rows if t > 1 else 0))
    return prefix, unit_rows


def make_item(item, q_lens, kv_lens, hq, group, window_left, rank):
    """Mirror of make_item(): the query tile of CTA `rank` and the union KV tile range."""
    pair_heads = group % 2 == 0
    head_units = hq // 2 if pair_heads else hq
    prefix, unit_rows = blocks_of(q_lens, pair_heads)
    total_units = prefix[-1]
    unit = total_units - 1 - item // head_units
    head_unit = item % head_units
    b = next(i for i in range(len(q_lens)) if prefix[i] <= unit < prefix[i + 1])
    t, n = q_lens[b], kv_lens[b]
    pos0 = n - t
    ur0 = (unit - prefix[b]) * unit_rows
    if pair_heads:
        tiles = [(2 * head_unit, ur0), (2 * head_unit + 1, ur0)]
    else:
        tiles = [(head_unit, ur0), (head_unit, ur0 + BM)]
    lo, hi, ranges = 1 << 30, -1, []
    for head, r0 in tiles:
        pmax = pos0 + min(r0 + BM - 1, t - 1)
        if r0 >= t or pmax < 0:
            ranges.append((0, -1))
            continue
        kmin = max(0, pos0 + r0 - window_left) if window_left >= 0 else 0
        ranges.append((kmin // BN, pmax // BN))
        lo, hi = min(lo, kmin // BN), max(hi, pmax // BN)
    return {"b": b, "pos0": pos0, "t": t, "tile": tiles[rank], "range": ranges[rank], "lo": lo,
            "n_tiles": hi - lo + 1 if hi >= 0 else 0, "total_items": total_units * head_units}


def visible(key, pos, window_left):
    return key <= pos and (window_left < 0 or key >= pos - window_left)


def test_every_block_and_head_is_covered_once_and_sees_its_keys():
    rng = random.Random(11)
    for _ in range(60):
        hkv = rng.choice([1, 2])
        group = rng.choice([1, 2, 3, 6])
        hq = hkv * group
        batch = rng.randint(1, 5)
        q_lens = [rng.choice([1, 2, 130, 300, rng.randint(2, 520)]) for _ in range(batch)]
        kv_lens = [max(0, t + rng.choice([0, 0, 200, -50, rng.randint(0, 900)])) for t in q_lens]
        window_left = rng.choice([-1, 0, 100, 255])
        n_items = make_item(0, q_lens, kv_lens, hq, group, window_left, 0)["total_items"] \
            if any(t > 1 for t in q_lens) else 0
        seen = set()
        for item in range(n_items):
            for rank in (0, 1):
                it = make_item(item, q_lens, kv_lens, hq, group, window_left, rank)
                head, r0 = it["tile"]
                if r0 < it["t"]:
                    key = (it["b"], r0, head)
                    assert key not in seen
                    seen.add(key)
                # every key a row of this tile may see lies in a tile the item walks
                for r in range(r0, min(r0 + BM, it["t"]), 37):
                    pos = it["pos0"] + r
                    for k in range(0, max(0, pos + 1)):
                        if visible(k, pos, window_left) and k < kv_lens[it["b"]]:
                            assert it["lo"] <= k // BN < it["lo"] + it["n_tiles"]
                            assert it["range"][0] <= k // BN <= it["range"][1]
        want = {(b, r0, h) for b, t in enumerate(q_lens) if t > 1
                for r0 in range(0, t, BM) for h in range(hq)}
        assert seen == want


def test_ring_phases_never_alias():
    """Event times of one cluster under the kernel's dependencies, with random
    durations: the waiter of phase k of a barrier always looks before phase k + 1 of
    the same barrier can complete (otherwise its parity wait would miss the phase)."""
    rng = random.Random(5)
    for _ in range(200):
        n = rng.randint(1, 40)  # KV tiles of the cluster's items, numbered g = 0 .. n - 1
        dur = lambda lo, hi: rng.uniform(lo, hi)  # noqa: E731
        s_done, p_done, pv_done, ld_done = [0.0] * n, [0.0] * n, [0.0] * n, [0.0] * n
        group_free = [0.0, 0.0]
        pv_issuer_free = 0.0
        s_issuer_free = 0.0
        s_seen, p_seen = [0.0] * n, [0.0] * n
        for g in range(n):
            # S of tile g: after the slot's last scores were taken (tile g - 2)
            start = max(s_issuer_free, ld_done[g - 2] if g >= 2 else 0.0)
            s_done[g] = start + dur(0.3, 1.0)
            s_issuer_free = start + dur(0.1, 0.6)
            # softmax group g % 2: after its tile before, scores ready, P buffer free
            w = g & 1
            s_seen[g] = max(group_free[w], s_done[g])
            ld_done[g] = s_seen[g] + dur(0.1, 0.4)
            p_start = max(ld_done[g], pv_done[g - 2] if g >= 2 else 0.0)
            p_done[g] = p_start + dur(0.5, 3.0)
            group_free[w] = p_done[g]
            # P V of tile g: in order, after P
            p_seen[g] = max(pv_issuer_free, p_done[g])
            pv_done[g] = p_seen[g] + dur(0.3, 1.0)
            pv_issuer_free = p_seen[g] + dur(0.1, 0.6)
        for g in range(n):
            # "scores ready" barrier g % 4: the group looks at phase g before S of tile g + 4
            if g + 4 < n:
                assert s_seen[g] <= s_done[g + 4]
            # "P ready" barrier g % 4: the issuer looks at tile g before tile g + 4 is ready
            if g + 4 < n:
                assert p_seen[g] <= p_done[g + 4]
            # hand-over word g % 4 of a row: read (with the scores of tile g) before the
            # maximum of tile g + 4 is written, which waits for P V of tile g + 2
            if g + 4 < n:
                assert ld_done[g] <= pv_done[g + 2]
