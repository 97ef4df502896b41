"""World-size-2 check of the KV-head sharding on CPU ranks (gloo): per-rank
attention over its own heads, the local ``wo`` product and the sum all-reduce
reproduce the unsharded layer, and the per-rank outputs concatenate to the
unsharded attention output bit for bit."""

from __future__ import annotations

import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cwm_b200.tp import Collectives, attention_out_proj, shard_cache_rows, shard_heads
from oracle import ref_paged_gqa_attention
from tests.helpers import make_problem

HQ, HKV, D, DIM = 12, 4, 32, 64


def _problem():
    return make_problem([1, 5, 1], [40, 23, 9], hq=HQ, hkv=HKV, d=D, page_size=8, seed=77,
                        dtype=torch.float32)


def _attend(p, q, rows, hq, hkv):
    k, v = torch.split(rows, [hkv * D, hkv * D], dim=1)
    shape = (-1, p.page_size, hkv, D)
    out, _ = ref_paged_gqa_attention(q, k.reshape(*shape), v.reshape(*shape), p.cu_seqlens_q,
                                     p.seqused_k, p.block_table, D**-0.5, 15)
    return out


def _worker(rank: int, world: int, port: int, queue) -> None:
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                            world_size=world)
    try:
        torch.manual_seed(5)
        wo = torch.randn(DIM, HQ * D)
        p = _problem()
        shard = shard_heads(rank, world, HQ, HKV)
        rows = shard_cache_rows(p.cache, shard, HKV, D)
        q_local = p.q[:, shard.q_begin : shard.q_end].contiguous()
        out_local = _attend(p, q_local, rows, shard.n_q, shard.n_kv)
        wo_local = wo[:, shard.q_begin * D : shard.q_end * D]
        h = attention_out_proj(out_local, wo_local, Collectives())
        gathered = [torch.empty_like(out_local) for _ in range(world)]
        dist.all_gather(gathered, out_local)
        if rank == 0:
            queue.put((h, torch.cat(gathered, dim=1)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharding_matches_unsharded():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for pr in procs:
        pr.start()
    h, out_cat = queue.get()
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    torch.manual_seed(5)
    wo = torch.randn(DIM, HQ * D)
    p = _problem()
    full = _attend(p, p.q, p.cache, HQ, HKV)
    # disjoint heads: the concatenation is the unsharded result, bit for bit
    assert torch.equal(out_cat, full)
    want = torch.nn.functional.linear(full.flatten(1, 2), wo)
    assert torch.allclose(h, want, rtol=1e-5, atol=1e-4)
