"""Host-side pieces of the generation engine, on the CPU: the block set against the
reference's own ``ISet``, the prefix trie against the reference's own ``Cache``
(both through ``tests/golden/engine_golden.json``, produced by
``tests/golden/make_engine_golden.py`` from the reference's modules), and the lane
scheduler's rules (``cwm/fastgen/generate.py:530-654,1016-1057``)."""

from __future__ import annotations

import json
import queue
import random
import sys
from pathlib import Path

import pytest
import torch

from cwm_b200.cache import RawCache
from cwm_b200.engine import Lane, LaneTable, Packet
from cwm_b200.hostcache import Cache, hashints
from cwm_b200.iset import ISet

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "golden"))
import make_engine_golden as gen  # noqa: E402


@pytest.fixture(scope="module")
def golden():
    return json.loads((ROOT / "golden" / "engine_golden.json").read_text())


class _ISetModule:
    ISet = ISet


# ------------------------------------------------------------------- block set
def test_block_set_replays_the_reference_results(golden):
    for entry in golden["iset"]:
        ops = gen.iset_script(entry["seed"])
        assert gen.run_iset(_ISetModule, ops) == entry["results"]


def test_block_set_properties():
    rng = random.Random(5)
    s, model = ISet(), set()
    for _ in range(2000):
        r = rng.random()
        if r < 0.4:
            a = rng.randrange(300)
            b = a + rng.randrange(20)
            s |= ISet.interval(a, b)
            model |= set(range(a, b))
        elif r < 0.6 and model:
            assert s.popleft() == min(model)
            model.remove(min(model))
        elif r < 0.8:
            n = rng.randrange(15)
            a, s = s.take(n)
            took = sorted(model)[:n]
            assert a.tolist() == took
            model -= set(took)
        else:
            e = rng.randrange(300)
            s.add(e)
            model.add(e)
        assert len(s) == len(model) and s.tolist() == sorted(model)
        runs = s.runs()
        assert all(a < b for a, b in runs)
        assert all(runs[i][1] < runs[i + 1][0] for i in range(len(runs) - 1))  # disjoint, not touching
    assert (5 in ISet.interval(3, 9)) and (9 not in ISet.interval(3, 9))
    assert len(ISet.interval(4, 4)) == 0
    with pytest.raises(ValueError):
        ISet.interval(-1, 3)
    with pytest.raises(IndexError):
        ISet().popleft()


# ------------------------------------------------------------------ prefix trie
class _CacheModule:
    """Adapter: lets the golden script drive this package's Cache."""

    RawCache = RawCache

    class Cache(Cache):
        def __init__(self, **kw):
            super().__init__(pin_memory=False, **kw)


def test_prefix_trie_replays_the_reference_results(golden):
    for entry in golden["cache"]:
        script = gen.cache_script(entry["seed"])
        assert gen.run_cache(_CacheModule, script) == entry["results"]


def test_prefix_trie_rules():
    c = Cache(limit_toks=40, node_len=4, page_len=4, pin_memory=False)
    gpu = RawCache([torch.zeros(32, 6)], [3, 3], 32)
    a = list(range(10))  # two whole pages + 2 tokens
    lane = c.prepare_lane(gpu, [7, 8, 9], a)
    assert lane.ready_count == 0 and len(lane.cpu_blocks) == 2 and c.num_nodes == 2
    assert lane.cpu_blocks[0].caches[0].shape == (4, 6)  # node_len rows, the cache's row layout
    assert list(lane.h2d_blocks()) == [] and [g for g, _ in lane.d2h_blocks()] == [7, 8]
    # pages inserted during this tick are not matchable yet (their K/V is not on the host)
    again = c.prepare_lane(gpu, [1, 2, 3], a)
    assert again.ready_count == 0 and c.num_nodes == 4
    c.tick()
    hit = c.prepare_lane(gpu, [4, 5, 6], a + [99, 98])  # third page is new
    assert hit.ready_count == 2 and len(hit.cpu_blocks) == 3
    assert hit.cpu_blocks[0] is lane.cpu_blocks[0] and hit.cpu_blocks[1] is lane.cpu_blocks[1]
    # no_insert stops at the first miss
    probe = c.prepare_lane(gpu, [1], [0, 1, 2, 3, 50, 51, 52, 53], no_insert=True)
    assert probe.ready_count == 1 and len(probe.cpu_blocks) == 1
    # a disabled cache hands back the device blocks only
    off = Cache(limit_toks=3, node_len=4, page_len=4, pin_memory=False)
    assert off.disabled and off.prepare_lane(gpu, [1, 2], a).cpu_blocks == []
    # eviction: least recently used leaves first, blocks return to the free list
    c.tick()
    for i in range(12):
        c.prepare_lane(gpu, [0], [1000 + i] * 4)
        c.tick()
    assert c.num_nodes > c.limit
    before = c.num_nodes
    c.maintain()
    assert c.num_nodes == int(0.75 * c.limit) and len(c.free_caches) == before - c.num_nodes


def test_hashints_is_stable_and_31_bit():
    assert hashints([1, 2, 3]) == hashints([1, 2, 3]) != hashints([3, 2, 1])
    assert 0 <= hashints(list(range(1000))) < 2**31


# --------------------------------------------------------------- lane scheduler
def _table(max_batch=4, nblocks=12, page=16):
    return LaneTable(max_batch, nblocks * page, page, vocab_size=100, device="cpu")


def _check_accounting(tb: LaneTable):
    owned = ISet()
    for i in range(tb.nactive):
        ln = tb.lane[i]
        assert ln.blocks == ln.blockset.tolist() or sorted(ln.blocks) == ln.blockset.tolist()
        for b in ln.blocks:
            assert b not in owned and b not in tb.free_blocks
            owned.add(b)
        assert tb.blktbl[i, : len(ln.blocks)].tolist() == ln.blocks
    assert len(owned) + len(tb.free_blocks) == tb.nblocks
    for i in range(tb.nactive, tb.max_batch):
        assert tb.lane[i].thread_id == "dead" and int(tb.seqlen[i]) == 0
        assert tb.blktbl[i].abs().sum() == 0


def _admit(tb, prompts, **kw):
    q = queue.Queue()
    for i, n in enumerate(prompts):
        q.put(Packet(thread_id=i, tokens=list(range(n))))
    q.put(None)
    eoq, added, cksum = tb.add_lanes(False, q, kw.get("max_gen"), kw.get("min_prefill", 0),
                                     kw.get("min_prefill_batch", 1))
    for i in range(tb.nactive, tb.nactive + added):  # what _prefill does for the table
        ln = tb.lane[i]
        tb.blktbl[i, : len(ln.blocks)] = torch.tensor(ln.blocks, dtype=torch.int)
        tb.seqlen[i] = len(ln) + 1
    tb.nactive += added
    return eoq, added, cksum


def test_admission_takes_blocks_with_head_room_and_parks_what_does_not_fit():
    tb = _table(max_batch=4, nblocks=24, page=16)
    eoq, added, cksum = _admit(tb, [10, 40, 200, 5])
    # blocks asked: (len + 128 + 15) // 16 -> 9, 11, then 21 > 4 free: parked, queue untouched after it
    assert added == 2 and not eoq and cksum != 0
    assert [len(tb.lane[i].blocks) for i in range(2)] == [9, 11]
    assert len(tb.parking) == 1 and len(tb.parking[0]) == 200
    assert tb.lane[0].blocks == list(range(9)) and tb.lane[1].blocks == list(range(9, 20))
    _check_accounting(tb)


def test_small_admissions_wait_while_decoding_has_work():
    tb = _table(max_batch=8, nblocks=64, page=16)
    _admit(tb, [30])
    q = queue.Queue()
    q.put(Packet(thread_id="x", tokens=[1, 2, 3]))
    eoq, added, _ = tb.add_lanes(False, q, None, min_prefill=512, min_prefill_batch=8)
    assert added == 0 and not eoq and len(tb.parking) == 1  # put back, blocks returned
    _check_accounting(tb)
    q.put(None)
    eoq, added, _ = tb.add_lanes(False, q, None, min_prefill=512, min_prefill_batch=8)
    assert eoq and added == 1  # the end of the queue lifts the wait


def test_kill_lane_moves_the_last_lane_into_the_slot():
    tb = _table(max_batch=4, nblocks=40, page=16)
    _admit(tb, [10, 20, 30])
    tb.top_p_lanes = {2}
    third = tb.lane[2]
    tb.kill_lane(0)
    assert tb.nactive == 2 and tb.lane[0] is third and tb.top_p_lanes == {0}
    assert int(tb.seqlen[0]) == 31 and tb.blktbl[0, : len(third.blocks)].tolist() == third.blocks
    _check_accounting(tb)
    tb.kill_lane(1, park=True)
    assert tb.nactive == 1 and len(tb.parking) == 1 and tb.parking[0].blocks == []
    _check_accounting(tb)


def test_prepare_lanes_grows_lanes_and_parks_the_shortest_when_blocks_run_out():
    tb = _table(max_batch=3, nblocks=30, page=16)
    _admit(tb, [10, 11, 12])  # 9 blocks each, 3 free
    for ln, grown in zip(tb.lane[:3], (140, 100, 143)):
        ln.tokens = list(range(grown - len(ln.prompt)))
    tb.prepare_lanes(sync_freq=10)
    # lanes of 140 and 143 tokens need a 10th block (150, 153 > 144); 100 + 10 fits
    assert [len(tb.lane[i].blocks) for i in range(3)] == [10, 9, 10]
    assert len(tb.free_blocks) == 1
    _check_accounting(tb)
    # grow all beyond their blocks; one block is free, so the shortest lanes are parked
    for ln, grown in zip(tb.lane[:3], (159, 150, 158)):
        ln.tokens = list(range(grown - len(ln.prompt)))
    tb.prepare_lanes(sync_freq=10)
    assert tb.nactive < 3 and len(tb.parking) == 3 - tb.nactive
    assert all(len(p) == n for p, n in zip(tb.parking, (150, 158)[: len(tb.parking)]))
    for i in range(tb.nactive):
        ln = tb.lane[i]
        assert len(ln) + 10 <= len(ln.blocks) * 16
    _check_accounting(tb)


def test_lane_from_packet_limits():
    ln = Lane.from_pkt(Packet(thread_id=1, tokens=[1] * 50, max_gen=30), max_seq=1000, max_gen=None)
    assert ln.maxlen == 80 and ln.prompt == [1] * 50 and ln.tokens == []
    assert Lane.from_pkt(Packet(thread_id=1, tokens=[1] * 50), 1000, None).maxlen == 1000
    assert Lane.from_pkt(Packet(thread_id=1, tokens=[1] * 50), 60, 30).maxlen == 60
