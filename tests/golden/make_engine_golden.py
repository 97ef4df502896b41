"""Generate ``engine_golden.json`` from the reference's block set and prefix cache.

Run where the reference checkout is readable::

    python tests/golden/make_engine_golden.py --reference /path/to/cwm

* ``cwm/fastgen/utils/iset.py`` (pure Python) is imported as it is and driven by a
  seeded script of operations; the resulting set contents, popped ids and splits
  are stored.
* ``cwm/fastgen/utils/cache.py`` is imported with its logging module
  (``utils/metrics.py``, which pulls in packages that are not installed here)
  replaced by a stub that records nothing, and ``Cache`` is driven without CUDA:
  stream creation is skipped and host blocks come from a pre-filled free list of
  plain CPU ``RawCache`` objects, so ``prepare_lane`` / ``tick`` / ``maintain`` run
  exactly the reference's trie code.  Stored per call: how many pages were ready,
  which host blocks the lane got (by serial number), and the node count.
"""

from __future__ import annotations

import argparse
import importlib
import json
import random
import sys
import types
from pathlib import Path

import torch


def iset_script(seed: int, n_ops: int = 300, universe: int = 600):
    """Operations as plain data, so that the test can replay them."""
    rng = random.Random(seed)
    ops = [("interval", rng.randrange(0, 50), rng.randrange(50, universe))]
    for _ in range(n_ops):
        kind = rng.choice(["add", "take", "popleft", "merge_interval", "take_put_back", "clear_some"])
        if kind == "add":
            ops.append(("add", rng.randrange(universe)))
        elif kind == "take":
            ops.append(("take", rng.randrange(0, 40)))
        elif kind == "popleft":
            ops.append(("popleft",))
        elif kind == "merge_interval":
            a = rng.randrange(universe)
            ops.append(("merge_interval", a, min(universe, a + rng.randrange(0, 30))))
        elif kind == "take_put_back":
            ops.append(("take_put_back", rng.randrange(0, 25)))
        else:
            ops.append(("merge_list", sorted(rng.sample(range(universe), rng.randrange(0, 12)))))
    return ops


def run_iset(iset_mod, ops):
    out = []
    s = iset_mod.ISet()
    for op in ops:
        if op[0] == "interval":
            s = iset_mod.ISet.interval(op[1], op[2])
            out.append(s.tolist())
        elif op[0] == "add":
            s.add(op[1])
            out.append(len(s))
        elif op[0] == "take":
            a, b = s.take(op[1])
            s = b
            out.append([a.tolist(), len(b)])
        elif op[0] == "popleft":
            out.append(s.popleft() if len(s) else None)
        elif op[0] == "merge_interval":
            s |= iset_mod.ISet.interval(op[1], op[2])
            out.append(len(s))
        elif op[0] == "take_put_back":
            a, b = s.take(op[1])
            b |= a
            s = b
            out.append(s.tolist())
        elif op[0] == "merge_list":
            o = iset_mod.ISet()
            for e in op[1]:
                o.add(e)
            s.merge(o)
            out.append(s.tolist())
    return out


def cache_script(seed: int):
    """Prompts built from a few shared prefixes, in rounds separated by ticks."""
    rng = random.Random(seed)
    page = 4
    stems = [[rng.randrange(100) for _ in range(page * rng.randrange(1, 5))] for _ in range(5)]
    rounds = []
    for _ in range(14):
        calls = []
        for _ in range(rng.randrange(1, 4)):
            toks = list(rng.choice(stems))
            toks += [rng.randrange(100) for _ in range(rng.randrange(0, 3 * page))]
            calls.append({"tokens": toks, "no_insert": rng.random() < 0.1})
        rounds.append(calls)
    return {"page_len": page, "node_len": page, "limit_pages": 18, "rounds": rounds}


def run_cache(cache_mod, script):
    class NoStreams(cache_mod.Cache):
        def _create_streams(self):
            pass

    c = NoStreams(limit_toks=script["limit_pages"] * script["page_len"],
                  node_len=script["node_len"], page_len=script["page_len"])
    serial = {}
    blocks = []
    for i in range(200):
        rc = cache_mod.RawCache([torch.zeros(script["node_len"], 2)], [1, 1], script["node_len"])
        serial[id(rc)] = i
        blocks.append(rc)
    c.free_caches = list(reversed(blocks))  # popped in serial order
    gpu = cache_mod.RawCache([torch.zeros(64, 2)], [1, 1], 64)
    out = []
    for calls in script["rounds"]:
        res = []
        for call in calls:
            lane = c.prepare_lane(gpu, [0, 1, 2], list(call["tokens"]), no_insert=call["no_insert"])
            res.append({"ready": lane.ready_count,
                        "blocks": [serial[id(b)] for b in lane.cpu_blocks],
                        "num_nodes": c.num_nodes})
        c.tick()
        c.maintain()
        out.append({"calls": res, "num_nodes_after_maintain": c.num_nodes,
                    "free": sorted(serial[id(b)] for b in c.free_caches)})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=str(Path(__file__).with_name("engine_golden.json")))
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    iset_mod = importlib.import_module("cwm.fastgen.utils.iset")
    stub = types.ModuleType("cwm.fastgen.utils.metrics")
    stub.dump = lambda *a, **k: None
    stub.recording = lambda: False
    sys.modules["cwm.fastgen.utils.metrics"] = stub
    cache_mod = importlib.import_module("cwm.fastgen.utils.cache")

    golden = {"iset": [], "cache": []}
    for seed in (1, 2, 3):
        ops = iset_script(seed)
        golden["iset"].append({"seed": seed, "results": run_iset(iset_mod, ops)})
    for seed in (11, 12):
        script = cache_script(seed)
        golden["cache"].append({"seed": seed, "results": run_cache(cache_mod, script)})
    Path(args.out).write_text(json.dumps(golden))
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
