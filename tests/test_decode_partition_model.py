"""Model of the decode kernel's work partition (cwm_b200/csrc/attn_decode.cu): the
flat list of 64-token tiles of all (sequence, KV head) segments is cut evenly over
the persistent CTAs; a segment that lies inside one CTA is written directly, any
other leaves one partial per CTA in slot 0 (segment began at or before the CTA's
range) or slot 1 (began inside it) and counts one arrival for the segment; the CTA
whose arrival is number ``c_last - c_first`` (counting from 0) merges exactly those
slots in CTA order.  This restates the index arithmetic in Python and checks its invariants on random
lengths; it guards the rule, not the CUDA code itself (the GPU tests do that)."""

from __future__ import annotations

import random


def partition(seg_tiles: list[int], grid: int):
    """Returns (direct, partial_writes): segments written directly, and the set of
    (cta, slot, segment) partials the persistent CTAs leave."""
    starts, total = [], 0
    for n in seg_tiles:
        starts.append(total)
        total += n
    per = (total + grid - 1) // grid if total else 0
    direct, partials, covered = set(), set(), [0] * len(seg_tiles)
    for cta in range(grid):
        g_begin = min(total, cta * per)
        g_end = min(total, g_begin + per)
        g = g_begin
        while g < g_end:
            seg = max(i for i, s in enumerate(starts) if s <= g and seg_tiles[i] > 0)
            seg_start, seg_end = starts[seg], starts[seg] + seg_tiles[seg]
            upto = min(seg_end, g_end)
            covered[seg] += upto - g
            if seg_start >= g_begin and seg_end <= g_end:
                direct.add(seg)
            else:
                slot = 0 if seg_start <= g_begin else 1
                assert (cta, slot) not in {(c, s) for c, s, _ in partials}, "slot reused"
                partials.add((cta, slot, seg))
            g = upto
    return direct, partials, covered, per, starts


def combine_reads(seg_tiles, grid, per, starts):
    """Slots the merging CTA of each split segment reads (CTAs c_first .. c_last)."""
    reads = set()
    for seg, n in enumerate(seg_tiles):
        if n == 0:
            continue
        s0, s1 = starts[seg], starts[seg] + n
        c_first, c_last = s0 // per, (s1 - 1) // per
        if c_first == c_last:
            continue
        for cta in range(c_first, c_last + 1):
            reads.add((cta, 0 if s0 <= cta * per else 1, seg))
    return reads


def test_partition_invariants_on_random_lengths():
    rng = random.Random(7)
    for _ in range(300):
        n_seg = rng.randint(1, 40)
        seg_tiles = [rng.choice([0, 0, 1, 2, 5, 17, 64, 300, 512]) for _ in range(n_seg)]
        grid = rng.choice([1, 2, 7, 296, 304])
        direct, partials, covered, per, starts = partition(seg_tiles, grid)
        # every tile of every segment is processed exactly once
        assert covered == seg_tiles
        nonempty = {i for i, n in enumerate(seg_tiles) if n > 0}
        split = {seg for _, _, seg in partials}
        # a segment is written directly or combined, never both, never neither
        assert direct | split == nonempty and not (direct & split)
        # the combine step reads exactly the partials that were written
        if per:
            assert combine_reads(seg_tiles, grid, per, starts) == partials
        # arrivals per split segment = number of CTAs the merge expects (c_last - c_first + 1)
        if per:
            for seg in split:
                s0, s1 = starts[seg], starts[seg] + seg_tiles[seg]
                arrivals = sum(1 for _, _, sg in partials if sg == seg)
                assert arrivals == (s1 - 1) // per - s0 // per + 1
        # at most two partials per CTA (its first and its last segment)
        for cta in range(grid):
            assert sum(1 for c, _, _ in partials if c == cta) <= 2
