"""Host-memory KV offload and prefix cache: ``DynCache`` and ``Cache`` of
``cwm/fastgen/utils/cache.py:172-483``.

A prompt's KV rows are kept in pinned host memory in blocks of ``node_len`` token
rows, indexed by a trie over pages of ``page_len`` tokens.  ``Cache.prepare_lane``
walks the trie with a new prompt: the pages it finds are blocks whose K/V need not
be recomputed (they are copied host -> device while the first layers run), the
pages it does not find get fresh blocks that the prefill call fills (device ->
host, layer by layer, behind the attention of each layer).  ``DynCache`` is the
``ModelCache`` handed to one prefill call; its ``page_in`` / ``page_out`` /
``cache_kv`` keep the reference's stream and event ordering
(``cache.py:211-280``): page-ins run on ``h2d_stream`` and are awaited by the
``cache_kv`` of their layer, page-outs run on ``d2h_stream`` behind an event
recorded on the compute stream.

The copies themselves differ from the reference: instead of one ``copy_`` per lane
and block and layer, each ``page_in`` / ``page_out`` is ONE kernel launch
(``cwm_block_copy``) that moves every block of that layer through addresses held in
a device table, reading or writing the pinned host blocks directly over the host
link.  The table is built once per ``DynCache``.
"""

from __future__ import annotations

import heapq
import itertools
import struct
from collections.abc import Iterable
from dataclasses import dataclass, field
from typing import Literal

import torch

from . import _lib
from .cache import ModelCache, RawCache


def hashints(vals: list[int]) -> int:
    """Hash of a list of ints as a non-negative integer below ``2**31``
    (``cwm/fastgen/utils/misc.py:9-16``: xxh32 of the values as little-endian
    uint32).  Falls back to BLAKE2 when xxhash is not installed; only equality of
    hashes within one process group matters."""
    data = struct.pack(f"<{len(vals)}I", *[v & 0xFFFFFFFF for v in vals])
    try:
        import xxhash

        return struct.unpack("<I", xxhash.xxh32_digest(data))[0] & 0x7FFFFFFF
    except ImportError:
        import hashlib

        return struct.unpack("<I", hashlib.blake2s(data, digest_size=4).digest())[0] & 0x7FFFFFFF


@dataclass
class DynCacheLane:
    """One lane of a prefill call: its device blocks and, position by position, the
    host blocks that mirror them; the first ``ready_count`` host blocks already hold
    valid K/V (host -> device), the others are to be filled (device -> host)."""

    gpu_blocks: list[int]
    cpu_blocks: list[RawCache]
    ready_count: int

    def h2d_blocks(self) -> Iterable[tuple[int, RawCache]]:
        return itertools.islice(zip(self.gpu_blocks, self.cpu_blocks), self.ready_count)

    def d2h_blocks(self) -> Iterable[tuple[int, RawCache]]:
        return itertools.islice(zip(self.gpu_blocks, self.cpu_blocks), self.ready_count, None)


@dataclass
class DynCache(ModelCache):
    """The cache object of one ``prefill()`` call: the device cache plus the paging
    of the lanes' blocks from and to host memory."""

    Mode = Literal["page_in", "page_out"]
    MODE_BITS = {"page_in": 1, "page_out": 2}

    gpu_cache: RawCache
    host_cache: "Cache"
    cache_lanes: list[DynCacheLane]
    h2d_events: list[tuple[torch.cuda.Event, int]] = field(default_factory=list)
    mode: int = 3
    _tables: dict = field(default_factory=dict, repr=False)

    def disable(self, mode: Mode) -> None:
        self.mode &= ~DynCache.MODE_BITS[mode]

    def enable(self, mode: Mode) -> None:
        self.mode |= DynCache.MODE_BITS[mode]

    # -- address tables: [n_layers, 2, n_blocks] (device side, host side) per direction
    def _table(self, direction: str) -> torch.Tensor | None:
        if direction in self._tables:
            return self._tables[direction]
        node_len = self.host_cache.node_len
        pairs = [p for lane in self.cache_lanes
                 for p in (lane.h2d_blocks() if direction == "h2d" else lane.d2h_blocks())]
        table = None
        if pairs:
            n_layers = len(self.gpu_cache.caches)
            rows = torch.empty((n_layers, 2, len(pairs)), dtype=torch.int64)
            for n in range(n_layers):
                dev = self.gpu_cache._cache(n)
                row_bytes = dev.stride(0) * dev.element_size()
                base = dev.data_ptr()
                for i, (gpu_block, cpu_block) in enumerate(pairs):
                    rows[n, 0, i] = base + gpu_block * node_len * row_bytes
                    rows[n, 1, i] = cpu_block._cache(n).data_ptr()
            table = rows.to(self.gpu_cache.caches[0].device)
        self._tables[direction] = table
        return table

    def _copy(self, n: int, direction: str, stream: torch.cuda.Stream) -> None:
        table = self._table(direction)
        if table is None:
            return
        dev = self.gpu_cache._cache(n)
        host = self.cache_lanes_host_layer(n)
        esz = dev.element_size()
        dst, src = (table[n, 0], table[n, 1]) if direction == "h2d" else (table[n, 1], table[n, 0])
        dst_pitch = (dev.stride(0) if direction == "h2d" else host.stride(0)) * esz
        src_pitch = (host.stride(0) if direction == "h2d" else dev.stride(0)) * esz
        code = _lib.load().cwm_block_copy(
            dst.data_ptr(), src.data_ptr(), table.shape[2], self.host_cache.node_len,
            dev.shape[1] * esz, dst_pitch, src_pitch, stream.cuda_stream)
        _lib.check(code, "block_copy")

    def cache_lanes_host_layer(self, n: int) -> torch.Tensor:
        """Layer ``n`` of any host block (all share one row layout)."""
        for lane in self.cache_lanes:
            if lane.cpu_blocks:
                return lane.cpu_blocks[0]._cache(n)
        raise RuntimeError("no host block in this call")

    def page_in(self, n: int) -> None:
        """Start the host -> device copy of layer ``n``'s ready blocks on the
        page-in stream and queue the event that ``cache_kv(n)`` will wait for."""
        if self.host_cache.disabled or not self.mode & 1:
            return
        assert all(nn < n for _, nn in self.h2d_events)
        stream = self.host_cache.h2d_stream
        with torch.cuda.stream(stream):
            self._copy(n, "h2d", stream)
        ev = torch.cuda.Event()
        ev.record(stream)
        self.h2d_events.append((ev, n))

    def page_out(self, n: int) -> None:
        """Start the device -> host copy of layer ``n``'s new blocks on the page-out
        stream, behind everything issued so far on the current stream (the layer's
        K/V writes)."""
        if self.host_cache.disabled or not self.mode & 2:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        stream = self.host_cache.d2h_stream
        with torch.cuda.stream(stream):
            ev.wait()
            self._copy(n, "d2h", stream)

    def host_cache_ready(self) -> torch.cuda.Event | None:
        """An event after which the host blocks written by this call are complete."""
        if self.host_cache.disabled:
            return None
        ev = torch.cuda.Event()
        ev.record(self.host_cache.d2h_stream)
        return ev

    def cache_kv(self, n: int) -> tuple[torch.Tensor, ...]:
        if not self.host_cache.disabled and (self.mode & 1):
            assert self.h2d_events and self.h2d_events[0][1] == n, \
                f"sync event is not available for layer {n}"
            ev, _ = self.h2d_events.pop(0)
            ev.wait()  # the page-in of this layer is done before it is read
        return self.gpu_cache.cache_kv(n)


@dataclass(eq=False)
class CacheNode:
    """One page of ``page_len`` tokens in the trie and the host block with its K/V."""

    toks_h: int
    toks: list[int]
    cache: RawCache
    clock: int
    node_id: int
    next: list["CacheNode"] = field(default_factory=list)

    def __lt__(self, other: "CacheNode") -> bool:
        # ties in the eviction order are broken by creation order, which is the same
        # on every tensor-parallel rank (object addresses are not)
        return self.node_id < other.node_id


@dataclass
class Cache:
    """Host cache for repeated prompt prefixes (``cache.py:303-483``)."""

    limit_toks: int
    node_len: int  # rows of a host block (= tokens of a device cache block on this rank)
    page_len: int  # tokens per trie page
    nodes: list[CacheNode] = field(default_factory=list)
    frozen: set[int] = field(default_factory=set)
    num_nodes: int = 0
    clock: int = 0
    next_id: int = 0
    downsize: float = 0.75
    limit: int = 0
    disabled: bool = False
    free_caches: list[RawCache] = field(default_factory=list)
    h2d_stream: torch.cuda.Stream | None = None
    d2h_stream: torch.cuda.Stream | None = None
    pin_memory: bool = True

    def __post_init__(self) -> None:
        self.limit = self.limit_toks // self.page_len
        self.disabled = self.limit == 0
        self._create_streams()

    def _create_streams(self) -> None:
        if torch.cuda.is_available():
            self.h2d_stream = torch.cuda.Stream()
            self.d2h_stream = torch.cuda.Stream()

    def tick(self) -> None:
        """Advance the clock: blocks inserted before this call become matchable."""
        self.frozen.clear()
        self.clock += 1

    def maintain(self) -> None:
        """Evict least-recently-used pages (deepest first among equals) until the
        trie holds ``downsize * limit`` pages, once it has grown past ``limit``."""
        if self.num_nodes <= self.limit:
            return
        to_evict = self.num_nodes - int(self.downsize * self.limit)
        entries: list[tuple[int, int, CacheNode, list[CacheNode]]] = []
        stack = [(n, self.nodes, 0) for n in self.nodes]
        while stack:
            node, siblings, depth = stack.pop()
            entries.append((node.clock, depth, node, siblings))
            stack.extend((child, node.next, depth - 1) for child in node.next)
        assert len(entries) == self.num_nodes
        self.num_nodes -= to_evict
        heapq.heapify(entries)
        for _ in range(to_evict):
            _, _, node, siblings = heapq.heappop(entries)
            # a page is never older than the pages below it, and deeper pages go first
            assert not node.next
            siblings.remove(node)
            self.free_caches.append(node.cache)

    def _new_block(self, gpu_cache: RawCache) -> RawCache:
        if self.free_caches:
            return self.free_caches.pop()
        return RawCache.build_like(gpu_cache, length=self.node_len, device="cpu",
                                   pin_memory=self.pin_memory)

    def prepare_lane(self, gpu_cache: RawCache, blocks: list[int], tokens: list[int],
                     no_insert: bool = False) -> DynCacheLane:
        """Match ``tokens`` page by page against the trie.  Pages found (and not
        inserted during this tick) give ready host blocks; from the first miss on,
        every further whole page gets a new trie node and a host block to fill.
        Returns the lane for a ``DynCache``."""
        if self.disabled:
            return DynCacheLane(blocks, [], 0)
        caches: list[RawCache] = []
        ready = 0
        inserting = False
        level = self.nodes
        for start in range(0, len(tokens) - self.page_len + 1, self.page_len):
            page = tokens[start : start + self.page_len]
            page_h = hashints(page)
            if not inserting:
                hit = next((n for n in level if id(n) not in self.frozen
                            and n.toks_h == page_h and n.toks == page), None)
                if hit is not None:
                    hit.clock = self.clock
                    caches.append(hit.cache)
                    level = hit.next
                    continue
                ready = len(caches)
                inserting = True
                if no_insert:
                    break
            node = CacheNode(page_h, page, self._new_block(gpu_cache), self.clock, self.next_id)
            level.append(node)
            self.frozen.add(id(node))
            caches.append(node.cache)
            level = node.next
            self.num_nodes += 1
            self.next_id += 1
        if not inserting:
            ready = len(caches)
        return DynCacheLane(blocks, caches, ready)

    def preallocate(self, gpu_cache: RawCache) -> None:
        """One pinned allocation for ``limit`` host blocks, cut into block views."""
        if self.disabled:
            return
        whole = RawCache.build_like(gpu_cache, length=self.node_len * self.limit, device="cpu",
                                    pin_memory=self.pin_memory)
        for i in range(self.limit):
            self.free_caches.append(whole.view(i * self.node_len, self.node_len))
