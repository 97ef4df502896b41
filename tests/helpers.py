"""Builders of seeded synthetic paged-attention problems shared by the tests."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PagedProblem:
    q: torch.Tensor            # [T, Hq, D]
    cache: torch.Tensor        # [rows, Hkv * 2 * D]  one layer, [K | V] per token row
    cu_seqlens_q: torch.Tensor  # int32 [B + 1]
    seqused_k: torch.Tensor    # int32 [B]
    block_table: torch.Tensor  # int32 [B, cols]
    page_size: int
    hq: int
    hkv: int
    d: int

    def kv_views(self, cache: torch.Tensor | None = None):
        c = self.cache if cache is None else cache
        k, v = torch.split(c, [self.hkv * self.d, self.hkv * self.d], dim=1)
        shape = (-1, self.page_size, self.hkv, self.d)
        return k.reshape(*shape), v.reshape(*shape)

    def to(self, device):
        return PagedProblem(
            self.q.to(device), self.cache.to(device), self.cu_seqlens_q.to(device),
            self.seqused_k.to(device), self.block_table.to(device), self.page_size, self.hq,
            self.hkv, self.d,
        )


def make_problem(
    q_lens: list[int],
    kv_lens: list[int],
    hq: int = 48,
    hkv: int = 8,
    d: int = 128,
    page_size: int = 256,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
    extra_pages: int = 3,
    table_cols: int | None = None,
) -> PagedProblem:
    """Random q and a cache whose pages are placed by a random permutation.

    Unused block-table entries are 0 (a valid page id), as in the reference
    engine, so a kernel that reads past a sequence's pages is not caught by an
    out-of-range id but by wrong results.
    """
    g = torch.Generator().manual_seed(seed)
    batch = len(q_lens)
    pages_per_seq = [(n + page_size - 1) // page_size for n in kv_lens]
    cols = max(pages_per_seq + [1]) if table_cols is None else table_cols
    n_pages = sum(pages_per_seq) + extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(batch, cols, dtype=torch.int32)
    it = iter(perm)
    for b, npg in enumerate(pages_per_seq):
        for c in range(npg):
            table[b, c] = next(it)
    cache = torch.randn(n_pages * page_size, hkv * 2 * d, generator=g).to(dtype)
    q = torch.randn(sum(q_lens), hq, d, generator=g).to(dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0).tolist()), dtype=torch.int32)
    return PagedProblem(
        q, cache, cu, torch.tensor(kv_lens, dtype=torch.int32), table, page_size, hq, hkv, d
    )
