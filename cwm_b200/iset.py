"""Ordered sets of small non-negative integers: the KV-cache block allocator.

Same interface and results as ``ISet`` of ``cwm/fastgen/utils/iset.py:282-323``
(``interval``, ``singleton``, ``add``, ``merge`` / ``|=``, ``take``, ``popleft``,
``clear``, ``tolist``, ``len``, iteration in ascending order), which the engine
uses for its free list and for the blocks of each lane
(``cwm/fastgen/generate.py:86,114-124,301,573,636``).  The reference keeps a
radix tree of bits; free block ids come and go in runs, so this version keeps a
sorted list of disjoint half-open runs ``[start, stop)`` and works on whole runs:
taking ``n`` blocks or returning a lane's blocks touches as many list entries as
there are runs, not as many as there are blocks.
"""

from __future__ import annotations

import bisect
from collections.abc import Iterator

_LIMIT = 1 << 32  # ids are below 2^32, as in the reference


class ISet:
    __slots__ = ("_starts", "_stops", "_count")

    def __init__(self, runs: list[tuple[int, int]] | None = None) -> None:
        self._starts: list[int] = []
        self._stops: list[int] = []
        self._count = 0
        for a, b in runs or []:
            self._insert_run(a, b)

    # ---------------------------------------------------------------- builders
    @staticmethod
    def interval(a: int, b: int) -> "ISet":
        """The ids ``a`` (inclusive) to ``b`` (exclusive); empty when ``b <= a``."""
        if a < 0:
            raise ValueError(f"{a=} must not be negative")
        if b > _LIMIT:
            raise ValueError(f"{b=} out of bounds (>{_LIMIT})")
        s = ISet()
        if b > a:
            s._starts, s._stops, s._count = [a], [b], b - a
        return s

    @staticmethod
    def singleton(elm: int) -> "ISet":
        return ISet.interval(elm, elm + 1)

    # ----------------------------------------------------------------- queries
    def __len__(self) -> int:
        return self._count

    def __bool__(self) -> bool:
        return self._count > 0

    def __contains__(self, elm: int) -> bool:
        i = bisect.bisect_right(self._starts, elm) - 1
        return i >= 0 and elm < self._stops[i]

    def __iter__(self) -> Iterator[int]:
        for a, b in zip(self._starts, self._stops):
            yield from range(a, b)

    def tolist(self) -> list[int]:
        return list(self)

    def runs(self) -> list[tuple[int, int]]:
        """The disjoint runs ``[start, stop)`` in ascending order."""
        return list(zip(self._starts, self._stops))

    def __eq__(self, other: object) -> bool:
        return isinstance(other, ISet) and self.runs() == other.runs()

    def __repr__(self) -> str:
        return f"ISet({self.runs()})"

    # --------------------------------------------------------------- mutation
    def _insert_run(self, a: int, b: int) -> None:
        """Union with ``[a, b)``; overlapping ids count once."""
        if b <= a:
            return
        if a < 0 or b > _LIMIT:
            raise ValueError(f"run [{a}, {b}) out of bounds")
        starts, stops = self._starts, self._stops
        # runs that touch or overlap [a, b): stop >= a and start <= b
        lo = bisect.bisect_left(stops, a)
        hi = bisect.bisect_right(starts, b)
        if lo < hi:
            removed = sum(stops[i] - starts[i] for i in range(lo, hi))
            a = min(a, starts[lo])
            b = max(b, stops[hi - 1])
            self._count -= removed
        starts[lo:hi] = [a]
        stops[lo:hi] = [b]
        self._count += b - a

    def add(self, elm: int) -> None:
        if elm >= _LIMIT:
            raise ValueError(f"{elm} out of bounds (>={_LIMIT})")
        self._insert_run(elm, elm + 1)

    def merge(self, other: "ISet") -> None:
        for a, b in zip(list(other._starts), list(other._stops)):
            self._insert_run(a, b)

    def __ior__(self, other: "ISet") -> "ISet":
        self.merge(other)
        return self

    def take(self, count: int) -> tuple["ISet", "ISet"]:
        """Split into the ``count`` smallest ids and the rest (both new sets; this
        set is unchanged).  With fewer than ``count`` ids, everything is taken."""
        taken, rest = ISet(), ISet()
        need = max(0, count)
        for a, b in zip(self._starts, self._stops):
            if need >= b - a:
                taken._starts.append(a)
                taken._stops.append(b)
                need -= b - a
            elif need > 0:
                taken._starts.append(a)
                taken._stops.append(a + need)
                rest._starts.append(a + need)
                rest._stops.append(b)
                need = 0
            else:
                rest._starts.append(a)
                rest._stops.append(b)
        taken._count = sum(b - a for a, b in zip(taken._starts, taken._stops))
        rest._count = self._count - taken._count
        return taken, rest

    def popleft(self) -> int:
        """Remove and return the smallest id."""
        if not self._count:
            raise IndexError("pop from an empty ISet")
        elm = self._starts[0]
        if self._stops[0] - elm == 1:
            del self._starts[0], self._stops[0]
        else:
            self._starts[0] = elm + 1
        self._count -= 1
        return elm

    def clear(self) -> None:
        self._starts, self._stops, self._count = [], [], 0
