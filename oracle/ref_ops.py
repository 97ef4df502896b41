"""CPU fp32 restatement of the reference hot path.  TEST INFRASTRUCTURE ONLY.

Every function cites the reference lines it follows (paths are relative to the
reference project root).  The functions take and return CPU torch tensors and
do their arithmetic in fp32, whatever the storage dtype of the inputs.
"""

from __future__ import annotations

import math

import torch


def ref_rope_freqs(
    head_dim: int,
    theta: float,
    scaled_rope: dict | None = None,
) -> torch.Tensor:
    """Rotary frequencies, ``cwm/fastgen/forward.py:1018-1047``.

    ``scaled_rope`` (optional) holds ``low_freq_factor``, ``high_freq_factor``,
    ``old_context_len`` and ``scale_factor`` for the wavelength-dependent
    rescaling of ``forward.py:1030-1045``.
    """
    pows = torch.arange(0, head_dim, 2).float() / head_dim
    freqs = 1.0 / (theta**pows)
    if scaled_rope is None:
        return freqs
    low = scaled_rope["low_freq_factor"]
    high = scaled_rope["high_freq_factor"]
    old_len = scaled_rope["old_context_len"]
    scaling = scaled_rope["scale_factor"]
    low_wavelen = old_len / low
    high_wavelen = old_len / high
    for idx, freq in enumerate(freqs):
        wavelen = 2 * math.pi / freq
        if wavelen > low_wavelen:
            freqs[idx] = freq / scaling
        if high_wavelen <= wavelen <= low_wavelen:
            x = old_len / wavelen - low
            x /= high - low
            freqs[idx] = (1 - x) * freq / scaling + x * freq
    return freqs


def ref_rope(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair rotary embedding, ``cwm/fastgen/kernels/rope.py:46-90``.

    ``x`` is ``[N, H, D]`` and is updated in place (rounded to its own dtype);
    the unrounded fp32 result is returned for tolerance checks.  The angle is
    ``float32(pos) * freq`` (``rope.py:58``) and pair ``i`` is ``(x[2i], x[2i+1])``
    (``rope.py:75-76``).
    """
    n, h, d = x.shape
    xf = x.float().reshape(n, h, d // 2, 2)
    angles = pos.to(torch.float32)[:, None] * freqs.to(torch.float32)[None, :]
    cos = torch.cos(angles)[:, None, :]
    sin = torch.sin(angles)[:, None, :]
    re, im = xf[..., 0], xf[..., 1]
    out = torch.stack((re * cos - im * sin, im * cos + re * sin), dim=-1)
    out = out.reshape(n, h, d)
    x.copy_(out.to(x.dtype))
    return out


def ref_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS normalisation, ``cwm/fastgen/kernels/rmsnorm.py:30-61``.

    Returns the fp32 value ``(x * rsqrt(mean(x^2) + eps)) * w`` in that
    association order (``rmsnorm.py:47,61``); the caller rounds it.
    """
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).sum(dim=-1, keepdim=True) / x.shape[-1] + eps)
    return (xf * rstd) * w.float()


def ref_paged_memcpy(
    src: torch.Tensor,
    dst: torch.Tensor,
    page_tbl: torch.Tensor,
    dst_pos: torch.Tensor,
    dst_shard: tuple[int, int] | None,
    src_batch: torch.Tensor | None,
    batch_size: torch.Tensor | int | None,
    page_size: int,
) -> None:
    """Scatter token rows into a paged destination,
    ``cwm/fastgen/kernels/paged_memcpy.py:56-87``.

    Row ``n`` goes to ``dst[page_tbl[b, pos // P] * P + pos % P]`` with
    ``b = src_batch[n]`` (``n`` when absent) and ``pos = dst_pos[n]``; rows at or
    beyond ``batch_size`` are skipped (``:57-61``), and with a shard ``(K, S)``
    only positions ``pos % S == K`` are kept, stored at ``pos // S`` (``:64-67``).
    """
    n_rows = src.shape[0]
    limit = n_rows if batch_size is None else int(batch_size)
    shard_idx, shard_cnt = dst_shard if dst_shard else (0, 1)
    for n in range(min(n_rows, limit)):
        pos = int(dst_pos[n])
        if shard_cnt > 1:
            if pos % shard_cnt != shard_idx:
                continue
            pos //= shard_cnt
        b = n if src_batch is None else int(src_batch[n])
        page = int(page_tbl[b, pos // page_size])
        dst[page * page_size + pos % page_size] = src[n]


def ref_paged_gqa_attention(
    q: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    seqused_k: torch.Tensor,
    block_table: torch.Tensor,
    softmax_scale: float,
    window_left: int = -1,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Varlen paged grouped-query attention as called at
    ``cwm/fastgen/forward.py:639-655`` (PARITY UNPINNED: the arithmetic of the
    reference lives in xformers' FlashAttention-3 binding).

    ``q`` is ``[T, Hq, D]``; ``key``/``value`` are ``[pages, P, Hkv, D]`` (views
    of the per-layer cache rows, ``forward.py:638,641-642``).  For sequence ``b``
    with ``t`` queries and ``n = seqused_k[b]`` keys, query ``j`` sits at absolute
    position ``p = n - t + j`` (``forward.py:511-519,525``) and attends keys
    ``max(0, p - window_left) .. p`` (all of ``0 .. p`` when ``window_left < 0``).
    Query head ``h`` reads KV head ``h // (Hq // Hkv)``.

    Returns ``(out fp32 [T, Hq, D], lse fp32 [Hq, T])``; a query with no visible
    key gives a zero row and ``lse = -inf``.
    """
    t_total, hq, d = q.shape
    n_pages, page_size, hkv, _ = key.shape
    group = hq // hkv
    out = torch.zeros(t_total, hq, d, dtype=torch.float32)
    lse = torch.full((hq, t_total), float("-inf"), dtype=torch.float32)
    cu = [int(v) for v in cu_seqlens_q]
    for b in range(len(cu) - 1):
        q0, q1 = cu[b], cu[b + 1]
        t = q1 - q0
        n = int(seqused_k[b])
        if t == 0 or n == 0:
            continue
        n_blocks = (n + page_size - 1) // page_size
        pages = block_table[b, :n_blocks].long()
        kb = key[pages].reshape(n_blocks * page_size, hkv, d)[:n].float()
        vb = value[pages].reshape(n_blocks * page_size, hkv, d)[:n].float()
        qb = q[q0:q1].float().reshape(t, hkv, group, d)
        # scores[h, g, j, k]
        s = torch.einsum("jhgd,khd->hgjk", qb, kb) * softmax_scale
        p = torch.arange(n - t, n)[:, None]
        k_idx = torch.arange(n)[None, :]
        visible = k_idx <= p
        if window_left >= 0:
            visible &= k_idx >= p - window_left
        s = s.masked_fill(~visible[None, None], float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        e = torch.exp(s - m_safe)
        l = e.sum(dim=-1, keepdim=True)
        prob = torch.where(l > 0, e / l.clamp_min(1e-38), torch.zeros_like(e))
        ob = torch.einsum("hgjk,khd->jhgd", prob, vb)
        out[q0:q1] = ob.reshape(t, hq, d)
        lse_b = (m_safe + torch.log(l)).squeeze(-1)  # log(0) = -inf for empty rows
        lse[:, q0:q1] = lse_b.reshape(hq, t)
    return out, lse


def ref_gqa_attention_layer(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    cache_row: torch.Tensor,
    q_seqpos: torch.Tensor,
    q_batch: torch.Tensor | None,
    actual_batch_size: torch.Tensor | int | None,
    freqs: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    seqused_k: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    window_left: int,
) -> torch.Tensor:
    """The GQA branch of the reference forward pass between the QKV projections
    and the output projection, ``cwm/fastgen/forward.py:608-656``.

    Order of operations as in the reference: rotate q and k in place
    (``:618-619``), write k then v rows to their pages (``:621-632``), then
    attend over the cache *including the rows just written* (``:638-655``).
    ``cache_row`` is one layer of the cache, ``[L, Hkv*(D+D)]`` with each row
    ``[K heads | V heads]`` (``cwm/fastgen/utils/cache.py:85-89,131-132``); it is
    updated in place.  ``xq`` and ``xk`` are updated in place as well.  Returns
    the fp32 attention output ``[T, Hq, D]``.
    """
    t_total, hq, d = xq.shape
    hkv = xk.shape[1]
    ref_rope(xq, q_seqpos, freqs)
    ref_rope(xk, q_seqpos, freqs)
    cache_k, cache_v = torch.split(cache_row, [hkv * d, hkv * d], dim=1)
    for x, c in ((xk, cache_k), (xv, cache_v)):
        ref_paged_memcpy(
            x.flatten(1, 2), c, block_table, q_seqpos, None, q_batch,
            actual_batch_size, page_size,
        )
    kv_shape = (-1, page_size, hkv, d)
    out, _ = ref_paged_gqa_attention(
        xq,
        cache_k.reshape(*kv_shape),
        cache_v.reshape(*kv_shape),
        cu_seqlens_q,
        seqused_k,
        block_table,
        d**-0.5,
        window_left,
    )
    return out


def ref_prefill_splits(seq_info: list[tuple[int, int]], max_prefill: int):
    """The prefill splitting loop of ``cwm/fastgen/generate.py:880-944`` with the model
    calls replaced by a record of their arguments: returns, per call, the token range
    ``(fst_tok, lst_tok)``, the first lane index and the ``seq_info`` slice passed to
    ``fwd.prefill``.  Log-probability handling (``:913-917``) is left out."""
    import bisect

    seq_info = list(seq_info)
    start_pos, total = [], 0
    for _, n in seq_info:
        start_pos.append(total)
        total += n
    calls = []
    fst_tok, lst_tok, fst_idx = 0, max_prefill, 0
    while lst_tok < total:
        lst_idx = bisect.bisect_left(start_pos, lst_tok, fst_idx)
        split_idx = lst_idx - 1
        cached, ntoks = seq_info[split_idx]
        new_ntoks = lst_tok - start_pos[split_idx]
        if new_ntoks == ntoks:
            new_ntoks -= 1
            lst_tok -= 1
        seq_info[split_idx] = (cached, new_ntoks)
        calls.append((fst_tok, lst_tok, fst_idx, list(seq_info[fst_idx:lst_idx])))
        cached += new_ntoks
        ntoks -= new_ntoks
        seq_info[split_idx] = (cached, ntoks)
        start_pos[split_idx] += new_ntoks
        fst_idx = split_idx
        fst_tok = lst_tok
        lst_tok += max_prefill
    calls.append((fst_tok, total, fst_idx, list(seq_info[fst_idx:])))
    return calls
