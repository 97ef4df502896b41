"""Tensor-parallel sharding of the attention path by KV head.

The reference shards attention over the ranks of a tensor-parallel group by
giving each rank a contiguous block of KV heads and the query heads that read
them (column-wise sharded ``wq``/``wk``/``wv``, local ``n_heads //= tp`` and
``n_kv_heads //= tp``: ``cwm/model/parallelize_transformer.py:88-102``).  Each
rank keeps cache rows ``[K_local | V_local]`` (``cwm/fastgen/utils/cache.py:85-89``);
block table and lengths are replicated.  Attention needs no communication; the
only collective is the sum all-reduce of the row-parallel ``wo`` output
(``cwm/fastgen/forward.py:763-768``), done here through ``torch.distributed``
(NCCL on GPUs, gloo in CPU tests).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    """Heads owned by one rank: half-open ranges of query and KV heads."""

    rank: int
    world: int
    q_begin: int
    q_end: int
    kv_begin: int
    kv_end: int

    @property
    def n_q(self) -> int:
        return self.q_end - self.q_begin

    @property
    def n_kv(self) -> int:
        return self.kv_end - self.kv_begin


def shard_heads(rank: int, world: int, n_heads: int, n_kv_heads: int) -> HeadShard:
    """Contiguous head block of ``rank`` among ``world`` ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a group of {world}")
    if n_kv_heads % world != 0 or n_heads % n_kv_heads != 0:
        raise ValueError(
            f"{n_heads} query / {n_kv_heads} KV heads cannot be split over {world} ranks"
        )
    kv_per = n_kv_heads // world
    group = n_heads // n_kv_heads
    return HeadShard(
        rank, world, rank * kv_per * group, (rank + 1) * kv_per * group,
        rank * kv_per, (rank + 1) * kv_per,
    )


def shard_cache_rows(full_rows: torch.Tensor, shard: HeadShard, n_kv_heads: int,
                     head_dim: int) -> torch.Tensor:
    """Local cache rows ``[K_local | V_local]`` cut out of full rows
    ``[K (all heads) | V (all heads)]`` (a copy; used to build test and bench
    inputs that agree across sharding degrees)."""
    k, v = torch.split(full_rows, [n_kv_heads * head_dim, n_kv_heads * head_dim], dim=1)
    sl = slice(shard.kv_begin * head_dim, shard.kv_end * head_dim)
    return torch.cat([k[:, sl], v[:, sl]], dim=1).contiguous()


class Collectives:
    """The subset of ``cwm/fastgen/utils/collectives.py`` that the attention path
    uses: a sum all-reduce over the tensor-parallel group."""

    def __init__(self, group: dist.ProcessGroup | None = None) -> None:
        self.group = group
        self.tp_size = dist.get_world_size(group)
        self.tp_rank = dist.get_rank(group)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x


def attention_out_proj(attn_out: torch.Tensor, wo_local: torch.Tensor,
                       coll: Collectives | None) -> torch.Tensor:
    """``F.linear(attn_out.flatten(1, 2), wo)`` followed by the all-reduce of
    ``forward.py:763-768``.  ``attn_out``: ``(T, Hq_local, D)``; ``wo_local``:
    ``(dim, Hq_local * D)``, this rank's column block of ``wo``."""
    h = torch.nn.functional.linear(attn_out.flatten(1, 2), wo_local)
    if coll is not None and coll.tp_size > 1:
        h = coll.all_reduce(h)
    return h
