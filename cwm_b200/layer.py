"""The GQA branch of the FastGen forward pass between the QKV projections and
the output projection (``cwm/fastgen/forward.py:608-656``), in two launches."""

from __future__ import annotations

import math

import torch

from .attention import mha_fwd, qkv_rope_kv_write, rope_kv_write
from .attn_bias import AttnBias
from .cache import ModelCache


def rope_freqs(
    head_dim: int, theta: float, scaled_rope: dict | None = None
) -> torch.Tensor:
    """Rotary frequencies as float32 ``(head_dim / 2,)`` on the CPU, computed with
    the same torch expression as ``cwm/fastgen/forward.py:1018-1047`` so that the
    angles agree to the bit.  ``scaled_rope`` may hold ``low_freq_factor``,
    ``high_freq_factor``, ``old_context_len`` and ``scale_factor``."""
    pows = torch.arange(0, head_dim, 2).float() / head_dim
    freqs = 1.0 / (theta**pows)
    if scaled_rope is None:
        return freqs
    low = scaled_rope["low_freq_factor"]
    high = scaled_rope["high_freq_factor"]
    old_len = scaled_rope["old_context_len"]
    scale = scaled_rope["scale_factor"]
    for i, f in enumerate(freqs):
        wavelen = 2 * math.pi / f
        if wavelen > old_len / low:
            freqs[i] = f / scale
        if old_len / high <= wavelen <= old_len / low:
            x = (old_len / wavelen - low) / (high - low)
            freqs[i] = (1 - x) * f / scale + x * f
    return freqs


def window_size_left(
    layer_id: int,
    n_layers: int,
    window_pattern: int,
    local_window: int | None,
    global_window: int | None = None,
    global_last_layer: bool = True,
) -> int:
    """``window_left`` of a layer under the interleaving rule of
    ``cwm/model/transformer.py:79-85,253-270``: a layer is global when
    ``layer_id % window_pattern == 0`` or, with ``global_last_layer``, when it is
    the last one; a window of ``w`` tokens gives ``w - 1``, no window gives -1."""
    is_global = (global_last_layer and layer_id == n_layers - 1) or layer_id % window_pattern == 0
    window = global_window if is_global else local_window
    return -1 if window is None else window - 1


def prefill_positions(
    seq_info: list[tuple[int, int]], device: torch.device | str | None = None
) -> tuple[torch.Tensor, torch.Tensor]:
    """``(q_batch, q_seqpos)`` for a prefill call (``forward.py:504-519``): for each
    new token its lane and its absolute position, given ``(cached, new)`` token
    counts per lane."""
    batch: list[int] = []
    pos: list[int] = []
    for i, (n0, n1) in enumerate(seq_info):
        batch.extend([i] * n1)
        pos.extend(range(n0, n0 + n1))
    return (
        torch.tensor(batch, dtype=torch.int32, device=device),
        torch.tensor(pos, dtype=torch.int32, device=device),
    )


def prefill_chunks(
    seq_info: list[tuple[int, int]], max_prefill: int
) -> list[tuple[int, int, int, list[tuple[int, int]]]]:
    """Cuts a prefill batch into calls of at most ``max_prefill`` new tokens, the way
    the reference engine does (``cwm/fastgen/generate.py:880-944``).

    ``seq_info`` holds ``(cached, new)`` token counts per lane, in the order in which
    the new tokens are concatenated.  Returns one entry per call:
    ``(first_token, last_token, first_lane, lane_seq_info)`` — the half-open range of
    the concatenated tokens to feed, the index of the first lane of the call, and the
    ``(cached, new)`` pairs of its lanes (a lane cut by the previous call continues
    with its cached count advanced).  As in the reference, a cut that would fall
    exactly on the end of a lane is moved one token back, so that every lane's last
    token is part of the call that also starts the next lane or ends the batch (its
    logits are the ones that are kept); a lane can therefore appear in a call with zero
    new tokens, which the attention ops treat as an empty sequence.
    """
    if max_prefill < 2:
        raise ValueError("max_prefill must be at least 2")
    info = [(int(c), int(n)) for c, n in seq_info]
    starts, total = [], 0
    for _, n in info:
        if n <= 0:
            raise ValueError("every lane needs at least one new token")
        starts.append(total)
        total += n
    calls = []
    first_tok, last_tok, first_lane = 0, max_prefill, 0
    while last_tok < total:
        # the lane that contains token last_tok - 1 ... the cut lies inside it or at its end
        lane = max(i for i in range(first_lane, len(info)) if starts[i] < last_tok)
        cached, n = info[lane]
        taken = last_tok - starts[lane]
        if taken == n:
            taken -= 1
            last_tok -= 1
        lanes = info[first_lane:lane] + [(cached, taken)]
        calls.append((first_tok, last_tok, first_lane, lanes))
        info[lane] = (cached + taken, n - taken)
        starts[lane] += taken
        first_lane, first_tok = lane, last_tok
        last_tok += max_prefill
    calls.append((first_tok, total, first_lane, info[first_lane:]))
    return calls


def gqa_attention(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    cache: ModelCache,
    layer_idx: int,
    attn_bias: AttnBias,
    q_seqpos: torch.Tensor,
    q_batch: torch.Tensor | None,
    actual_batch_size: torch.Tensor | None,
    freqs: torch.Tensor,
    window_left: int,
) -> torch.Tensor:
    """Rotary embedding, KV-cache write and attention for one layer.

    ``xq``: ``(T, Hq, D)``, ``xk``/``xv``: ``(T, Hkv, D)`` straight from the QKV
    projections.  ``xq`` and ``xk`` are rotated in place, the new K/V rows are
    written at ``q_seqpos`` through ``attn_bias.block_tables`` (lane ``q_batch[n]``,
    or ``n`` in decode), then every query attends over its sequence's pages
    *including* the rows just written.  Returns ``(T, Hq, D)``.
    """
    cache_k, cache_v = cache.cache_kv(layer_idx)
    hkv, d = xk.shape[1], xk.shape[2]
    page = attn_bias.page_size
    rope_kv_write(
        xq, xk, xv, cache_k, cache_v, q_seqpos, freqs, attn_bias.block_tables, q_batch,
        actual_batch_size, page,
    )
    cache.page_out(layer_idx)
    out, _ = mha_fwd(
        query=xq,
        key=cache_k.reshape(-1, page, hkv, d),
        value=cache_v.reshape(-1, page, hkv, d),
        cu_seqlens_q=attn_bias.q_seqinfo.seqstart,
        cu_seqlens_k=None,
        seqused_k=attn_bias.k_seqinfo.seqlen,
        leftpad_k=None,
        max_seqlen_q=attn_bias.q_seqinfo.max_seqlen,
        max_seqlen_k=attn_bias.k_seqinfo.max_seqlen,
        p=0,
        block_table=attn_bias.block_tables,
        softmax_scale=d**-0.5,
        is_causal=True,
        window_left=window_left,
        window_right=-1,
    )
    return out


def gqa_attention_packed(
    qkv: torch.Tensor,
    n_heads: int,
    n_kv_heads: int,
    cache: ModelCache,
    layer_idx: int,
    attn_bias: AttnBias,
    q_seqpos: torch.Tensor,
    q_batch: torch.Tensor | None,
    actual_batch_size: torch.Tensor | None,
    freqs: torch.Tensor,
    window_left: int,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``gqa_attention`` for the packed output ``qkv = x @ [wq | wk | wv]^T`` of one
    stacked projection, ``(T, (Hq + 2 Hkv) * D)``: same result as splitting it into
    ``xq``, ``xk``, ``xv`` and calling ``gqa_attention``, without the copies.  ``qkv``
    may live in pinned host memory and ``out`` may name a pinned host tensor for the
    result: the two kernels then move the step's inputs and outputs across the host
    link themselves."""
    cache_k, cache_v = cache.cache_kv(layer_idx)
    page = attn_bias.page_size
    d = qkv.shape[1] // (n_heads + 2 * n_kv_heads)
    xq = qkv_rope_kv_write(
        qkv, n_heads, n_kv_heads, cache_k, cache_v, q_seqpos, freqs, attn_bias.block_tables,
        q_batch, actual_batch_size, page,
    )
    cache.page_out(layer_idx)
    out, _ = mha_fwd(
        xq, cache_k.reshape(-1, page, n_kv_heads, d), cache_v.reshape(-1, page, n_kv_heads, d),
        attn_bias.q_seqinfo.seqstart, None, attn_bias.k_seqinfo.seqlen, None,
        attn_bias.q_seqinfo.max_seqlen, attn_bias.k_seqinfo.max_seqlen, 0,
        attn_bias.block_tables, d**-0.5, True, window_left, -1, out=out,
    )
    return out
