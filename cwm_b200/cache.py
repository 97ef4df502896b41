"""Paged KV-cache storage with the layout of ``cwm/fastgen/utils/cache.py``.

One 2-D tensor per layer, ``[tokens, Hkv * (D + D)]``; a token row holds the keys
of all local KV heads followed by their values (``cache.py:85-89``).  Pages are
consecutive ranges of ``page_size`` rows.  The kernels address the K and V halves
as strided views of these rows, so the layout is part of the drop-in contract.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


class ModelCache:
    """Interface of ``cache.py:28-45``: per-layer K/V access plus paging hooks."""

    def cache_kv(self, n: int) -> tuple[torch.Tensor, ...]:
        raise NotImplementedError

    def page_in(self, n: int) -> None:
        """Hook: bring layer ``n`` from host to device (no-op for a device cache)."""

    def page_out(self, n: int) -> None:
        """Hook: copy layer ``n`` from device to host (no-op for a device cache)."""


@dataclass
class RawCache(ModelCache):
    caches: list[torch.Tensor]
    split: list[int]
    length: int
    start: int = 0

    @staticmethod
    def build_dims(
        n_layers: int,
        n_kv_heads: int,
        head_dim: int,
        length: int,
        device: torch.device | str | None = None,
        dtype: torch.dtype | None = None,
    ) -> "RawCache":
        """Zero-filled cache of ``length`` token rows per layer for a GQA model
        with ``n_kv_heads`` local KV heads."""
        width = n_kv_heads * head_dim
        return RawCache(
            [torch.zeros((length, 2 * width), device=device, dtype=dtype) for _ in range(n_layers)],
            [width, width],
            length,
        )

    @staticmethod
    def build(
        model,
        length: int,
        device: torch.device | str | None = None,
        dtype: torch.dtype | None = None,
    ) -> "RawCache":
        """``RawCache.build`` of ``cache.py:57-97`` for GQA models: ``model`` needs
        ``n_layers``, ``qk_head_dim``, ``head_dim``, ``kv_lora_rank`` and
        ``layers[0].attention.n_kv_heads``."""
        if getattr(model, "kv_lora_rank", 0) > 0:
            raise NotImplementedError("latent-attention (MLA) caches are outside this package")
        if model.qk_head_dim != model.head_dim:
            raise NotImplementedError("K and V head dimensions must be equal")
        return RawCache.build_dims(
            model.n_layers, model.layers[0].attention.n_kv_heads, model.head_dim, length,
            device, dtype,
        )

    @staticmethod
    def build_like(
        other: "RawCache",
        length: int,
        device: str | None = None,
        pin_memory: bool = False,
    ) -> "RawCache":
        """A cache with the row layout of ``other`` in one allocation, optionally
        in pinned host memory (``cache.py:99-121``)."""
        first = other.caches[0]
        storage = torch.empty(
            (len(other.caches), length, first.shape[1]),
            dtype=first.dtype,
            device=device if device is not None else first.device,
            pin_memory=pin_memory,
        )
        return RawCache([storage[i] for i in range(len(other.caches))], other.split, length)

    def _cache(self, n: int) -> torch.Tensor:
        return self.caches[n][self.start : self.start + self.length]

    def cache_kv(self, n: int) -> tuple[torch.Tensor, ...]:
        """``(cache_k, cache_v)``: column views ``[length, Hkv * D]`` of layer ``n``."""
        return torch.split(self._cache(n), self.split, dim=1)

    def view(self, start: int, length: int) -> "RawCache":
        """A window of ``length`` rows starting at ``start`` over the same storage."""
        if start + length > self.length:
            raise ValueError("view exceeds the cache")
        return RawCache(self.caches, self.split, start=self.start + start, length=length)

    def bytes_per_token(self) -> int:
        if not self.caches:
            return 0
        first = self.caches[0]
        return len(self.caches) * first[0].numel() * first.element_size()

    def clear(self) -> None:
        for c in self.caches:
            c.zero_()
