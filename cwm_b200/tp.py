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


class _RawCuda:
    """Raw device memory as an object ``torch.as_tensor`` can wrap (uint8)."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
        }


class PeerAllReduce:
    """The node-local all-reduce kernel of this package (``cwm_allreduce``) with its
    buffers: the counterpart of the reference's ``CustomAllreduce``
    (``cwm/fastgen/utils/collectives.py:11-15,39-45``).

    Each rank allocates a scratch buffer, two result buffers and a flag array through
    ``cwm_peer_alloc`` and maps the other ranks' buffers through CUDA IPC (the ranks
    are processes on one node; the 64-byte handles travel through the process group).
    ``all_reduce(x)`` takes any contiguous bf16 / fp16 device tensor and returns the
    sum as a view of one of the two result buffers, which alternate from call to
    call: a result stays valid until the second call after it.  ``close`` is a
    collective call: every rank unmaps its peers, all meet at a barrier, then each
    frees its own buffers, so that no rank releases memory that a peer still maps.
    """

    def __init__(self, group: dist.ProcessGroup | None, device: torch.device,
                 max_bytes: int = 8 << 20) -> None:
        import ctypes

        from . import _lib

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the peer all-reduce serves at most 8 ranks of one node")
        self.device = device
        self.max_bytes = max_bytes
        self._lib = _lib.load()
        # scratch, result 0, result 1, flags
        sizes = [max_bytes, max_bytes, max_bytes, self._lib.cwm_allreduce_flag_ints() * 4]
        self._own: list[int] = []
        self._peers: list[int] = []
        self._tables = []
        with torch.cuda.device(device):
            for nbytes in sizes:
                ptr = ctypes.c_void_p()
                handle = ctypes.create_string_buffer(64)
                _lib.check(self._lib.cwm_peer_alloc(nbytes, ctypes.byref(ptr), handle), "peer_alloc")
                self._own.append(ptr.value)
                gathered: list = [None] * self.world
                dist.all_gather_object(gathered, bytes(handle.raw), group=group)
                ptrs = []
                for p, h in enumerate(gathered):
                    if p == self.rank:
                        ptrs.append(ptr.value)
                        continue
                    mapped = ctypes.c_void_p()
                    _lib.check(self._lib.cwm_peer_open(ctypes.create_string_buffer(h, 64),
                                                       ctypes.byref(mapped)), "peer_open")
                    self._peers.append(mapped.value)
                    ptrs.append(mapped.value)
                self._tables.append(ctypes_array(ptrs))
            self._results = [torch.as_tensor(_RawCuda(self._own[1 + i], max_bytes), device=device)
                             for i in range(2)]
            self._epoch = torch.tensor([1, 0], dtype=torch.int32, device=device)
        self._calls = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def supports(self, x: torch.Tensor) -> bool:
        return (x.dtype in (torch.bfloat16, torch.float16) and x.is_contiguous()
                and x.numel() % (8 * self.world) == 0 and x.data_ptr() % 16 == 0
                and x.numel() * x.element_size() <= self.max_bytes)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        from . import _lib
        from .kernels import _DTYPES, _stream

        if not self.supports(x):
            raise ValueError("the peer all-reduce takes contiguous, 16-byte aligned bf16 or fp16 "
                             "tensors whose size splits into 16-byte vectors over the ranks and "
                             "fits its buffers")
        which = self._calls & 1
        self._calls += 1
        code = _lib.load().cwm_allreduce(
            x.data_ptr(), self._tables[0], self._tables[1 + which], self._tables[3],
            self._epoch.data_ptr(), x.numel(), _DTYPES[x.dtype], self.rank, self.world, _stream(x))
        _lib.check(code, "allreduce")
        nbytes = x.numel() * x.element_size()
        return self._results[which][:nbytes].view(x.dtype).view(x.shape)

    def supports_add_rmsnorm(self, x: torch.Tensor, h: torch.Tensor, w: torch.Tensor) -> bool:
        return (x.dim() == 2 and self.supports(x) and x.shape[0] % self.world == 0
                and h.shape == x.shape and h.dtype == x.dtype and h.is_contiguous()
                and w.dtype == x.dtype and w.numel() == x.shape[1] and w.is_contiguous()
                and (x.shape[1] * x.element_size()) % 16 == 0
                and x.shape[1] * x.element_size() <= 32768
                and h.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def all_reduce_add_rmsnorm(self, x: torch.Tensor, h: torch.Tensor, w: torch.Tensor,
                               eps: float) -> torch.Tensor:
        """``rmsnorm(h + all_reduce(x), w)`` in one kernel (``cwm_allreduce_add_rmsnorm``).
        Updates this rank's rows of ``h`` (rows ``rank * T / world`` onwards) in place
        and leaves the others alone: the caller keeps the residual stream sharded by
        rows.  Returns the normalised activations of all rows as a view of a result
        buffer (valid until the second call after this one)."""
        from . import _lib
        from .kernels import _DTYPES, _stream

        if not self.supports_add_rmsnorm(x, h, w):
            raise ValueError("all_reduce_add_rmsnorm: see PeerAllReduce.supports_add_rmsnorm")
        which = self._calls & 1
        self._calls += 1
        code = _lib.load().cwm_allreduce_add_rmsnorm(
            x.data_ptr(), h.data_ptr(), w.data_ptr(), self._tables[0], self._tables[1 + which],
            self._tables[3], self._epoch.data_ptr(), x.shape[0], x.shape[1], float(eps),
            _DTYPES[x.dtype], self.rank, self.world, _stream(x))
        _lib.check(code, "allreduce_add_rmsnorm")
        nbytes = x.numel() * x.element_size()
        return self._results[which][:nbytes].view(x.dtype).view(x.shape)

    def close(self) -> None:
        """Collective: unmap the peers' buffers, barrier, free the own buffers."""
        if not self._own:
            return
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for ptr in self._peers:
                self._lib.cwm_peer_close(ptr)
            self._peers = []
            dist.barrier(group=self.group)
            self._results = []
            for ptr in self._own:
                self._lib.cwm_peer_free(ptr)
            self._own = []
        self._tables = []


def ctypes_array(values: list[int]):
    import ctypes

    return (ctypes.c_uint64 * len(values))(*values)


class Collectives:
    """The subset of ``cwm/fastgen/utils/collectives.py`` that the attention path
    uses: a sum all-reduce over the tensor-parallel group, through the node-local
    peer-memory kernel when ``peer`` is given and the tensor qualifies (the
    reference's rule: its custom all-reduce below 8 MiB, ``collectives.py:73-88``),
    through the process group's all-reduce (NCCL on GPUs, gloo in CPU tests)
    otherwise.  With the peer kernel the result is a view of a buffer that the
    second next call overwrites; with the process group it is ``x`` itself."""

    def __init__(self, group: dist.ProcessGroup | None = None,
                 peer: PeerAllReduce | None = None) -> None:
        self.group = group
        self.tp_size = dist.get_world_size(group)
        self.tp_rank = dist.get_rank(group)
        self.peer = peer

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.peer is not None and self.peer.supports(x):
            return self.peer.all_reduce(x)
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x

    def linear_all_reduce(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``all_reduce(F.linear(x, weight))`` (``forward.py:763-768,782-785``)."""
        return self.all_reduce(torch.nn.functional.linear(x, weight))

    def fuses_add_rmsnorm(self, rows: int, dim: int, dtype: torch.dtype) -> bool:
        """Whether ``linear_all_reduce_add_rmsnorm`` runs as one kernel for products of
        this shape (then only this rank's rows of the residual stream are kept current)."""
        return (self.peer is not None and rows % self.tp_size == 0 and rows > 0
                and dtype in (torch.bfloat16, torch.float16)
                and (dim * 2) % 16 == 0 and dim * 2 <= 32768
                and rows * dim * 2 <= self.peer.max_bytes and (rows * dim) % (8 * self.tp_size) == 0)

    def linear_all_reduce_add_rmsnorm(self, x: torch.Tensor, weight: torch.Tensor,
                                      h: torch.Tensor, w: torch.Tensor, eps: float,
                                      fused: bool) -> torch.Tensor:
        """``rms_norm(h + all_reduce(F.linear(x, weight)), w)`` with ``h`` updated in
        place (``forward.py:763-772,782-789``).  ``fused``: through the peer-memory
        kernel that does all three (the caller asked ``fuses_add_rmsnorm`` first and
        keeps to one choice for a whole pass, because the fused form keeps only this
        rank's rows of ``h`` current)."""
        from .kernels import add_rmsnorm

        y = torch.nn.functional.linear(x, weight)
        if fused:
            return self.peer.all_reduce_add_rmsnorm(y, h, w, eps)
        return add_rmsnorm(h, self.all_reduce(y), w, eps)

    def close(self) -> None:
        if self.peer is not None:
            self.peer.close()
            self.peer = None


def attention_out_proj(attn_out: torch.Tensor, wo_local: torch.Tensor,
                       coll: Collectives | None) -> torch.Tensor:
    """``F.linear(attn_out.flatten(1, 2), wo)`` followed by the all-reduce of
    ``forward.py:763-768``.  ``attn_out``: ``(T, Hq_local, D)``; ``wo_local``:
    ``(dim, Hq_local * D)``, this rank's column block of ``wo``."""
    h = torch.nn.functional.linear(attn_out.flatten(1, 2), wo_local)
    if coll is not None and coll.tp_size > 1:
        h = coll.all_reduce(h)
    return h
