"""Metadata holder for paged, variable-length causal attention.

Stands in for ``xformers.ops.fmha.attn_bias.
PagedBlockDiagonalCausalWithOffsetPaddedKeysMask`` as far as
``cwm/fastgen/forward.py`` uses it (``forward.py:12-14,70-77,97,115,131,502,
511,525,626,631,638,643-650,875-887``): construction from Python lists of
lengths, device tensors that the decode loop mutates in place between graph
replays, and the Python-side copies of the lengths.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class SeqLenInfo:
    """Query side: ``seqstart`` is the int32 exclusive prefix sum ``(B + 1,)``."""

    seqstart: torch.Tensor
    seqstart_py: list[int]
    max_seqlen: int
    min_seqlen: int

    def to(self, device: torch.device | str) -> None:
        """Move the tensor to ``device`` in place (the object keeps its identity)."""
        self.seqstart = self.seqstart.to(device, non_blocking=True)

    @classmethod
    def from_seqlens(cls, seqlens: list[int], device: torch.device | str | None) -> "SeqLenInfo":
        starts = [0]
        for n in seqlens:
            starts.append(starts[-1] + int(n))
        return cls(
            seqstart=torch.tensor(starts, dtype=torch.int32, device=device),
            seqstart_py=starts,
            max_seqlen=max(seqlens) if seqlens else 0,
            min_seqlen=min(seqlens) if seqlens else 0,
        )


@dataclass
class PaddedSeqLenInfo:
    """Key side: ``seqlen`` is the int32 number of keys per sequence ``(B,)``.

    ``seqlen`` is what the decode loop overwrites before every graph replay
    (``forward.py:131``); the kernels read it on the device.
    """

    seqlen: torch.Tensor
    seqlen_py: list[int]
    max_seqlen: int
    min_seqlen: int
    padding: int

    def to(self, device: torch.device | str) -> None:
        self.seqlen = self.seqlen.to(device, non_blocking=True)

    @classmethod
    def from_seqlens(
        cls, seqlens: list[int], padding: int, device: torch.device | str | None
    ) -> "PaddedSeqLenInfo":
        return cls(
            seqlen=torch.tensor([int(n) for n in seqlens], dtype=torch.int32, device=device),
            seqlen_py=[int(n) for n in seqlens],
            max_seqlen=max(seqlens) if seqlens else 0,
            min_seqlen=min(seqlens) if seqlens else 0,
            padding=padding,
        )


@dataclass
class PagedBlockDiagonalCausalWithOffsetPaddedKeysMask:
    """Block-diagonal causal mask over paged keys: sequence ``b`` has
    ``q_seqinfo`` queries that end at key ``k_seqinfo.seqlen[b] - 1`` (bottom-right
    aligned), and its keys live in the pages listed in ``block_tables[b]``."""

    q_seqinfo: SeqLenInfo
    k_seqinfo: PaddedSeqLenInfo
    block_tables: torch.Tensor
    page_size: int

    @classmethod
    def from_seqlens(
        cls,
        q_seqlen: list[int],
        kv_seqlen: list[int],
        block_tables: torch.Tensor,
        page_size: int,
    ) -> "PagedBlockDiagonalCausalWithOffsetPaddedKeysMask":
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must have the same length")
        if block_tables.ndim != 2 or block_tables.shape[0] != len(q_seqlen):
            raise ValueError("block_tables must be (len(q_seqlen), cols)")
        if block_tables.dtype != torch.int32:
            raise ValueError("block_tables must be an int32 tensor")
        device = block_tables.device
        return cls(
            q_seqinfo=SeqLenInfo.from_seqlens(q_seqlen, device),
            k_seqinfo=PaddedSeqLenInfo.from_seqlens(
                kv_seqlen, block_tables.shape[1] * page_size, device
            ),
            block_tables=block_tables,
            page_size=page_size,
        )


AttnBias = PagedBlockDiagonalCausalWithOffsetPaddedKeysMask
