"""CPU fp32 restatement of a decode step and of a prefill call of the GQA decoder.
TEST INFRASTRUCTURE ONLY.  Follows the GQA path of ``cwm/fastgen/forward.py:467-821`` for an unsharded
model: embedding, then per layer RMSNorm -> q/k/v projections -> rotary embedding
-> KV-cache write -> paged attention -> output projection -> residual ->
RMSNorm -> SwiGLU -> residual, then the final norm and the vocabulary projection.
Weights are given as a dict of fp32 tensors; activations stay fp32 throughout
(the GPU path rounds to bf16 between ops, which the caller's tolerance covers).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .ref_ops import ref_gqa_attention_layer, ref_rmsnorm


def ref_decode_step(weights: dict, tokens: torch.Tensor, seqlen: torch.Tensor,
                    block_tbl: torch.Tensor, caches: list[torch.Tensor], freqs: torch.Tensor,
                    n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, eps: float,
                    nactive: int | None = None) -> torch.Tensor:
    """``caches[i]`` is layer ``i``'s ``[rows, Hkv * 2 * D]`` cache (updated in place);
    ``seqlen`` counts the token being fed (``forward.py:525``: position = seqlen - 1).
    Returns fp32 logits ``(batch, vocab)``."""
    batch = tokens.shape[0]
    pos = (seqlen - 1).to(torch.int32)
    cu = torch.arange(batch + 1, dtype=torch.int32)
    h = F.embedding(tokens.long(), weights["tok_embeddings"])
    for i, layer in enumerate(weights["layers"]):
        x = ref_rmsnorm(h, layer["attention_norm"], eps)
        xq = F.linear(x, layer["wq"]).view(batch, n_heads, head_dim)
        xk = F.linear(x, layer["wk"]).view(batch, n_kv_heads, head_dim)
        xv = F.linear(x, layer["wv"]).view(batch, n_kv_heads, head_dim)
        attn = ref_gqa_attention_layer(
            xq, xk, xv, caches[i], pos, None, nactive, freqs, cu, seqlen.to(torch.int32),
            block_tbl, page_size, layer["window_left"],
        )
        h = h + F.linear(attn.flatten(1, 2), layer["wo"])
        x = ref_rmsnorm(h, layer["ffn_norm"], eps)
        x1, x3 = F.linear(x, layer["w13"]).chunk(2, dim=1)
        h = h + F.linear(F.silu(x1) * x3, layer["w2"])
    h = ref_rmsnorm(h, weights["norm"], eps)
    return F.linear(h, weights["output"])


def ref_prefill(weights: dict, token_values: torch.Tensor, seq_info: list[tuple[int, int]],
                block_tbl: torch.Tensor, caches: list[torch.Tensor], freqs: torch.Tensor,
                n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, eps: float,
                all_rows: bool = False) -> torch.Tensor:
    """``prefill`` of ``cwm/fastgen/forward.py:824-926`` for an unsharded GQA model:
    positions ``n0 .. n0 + n1 - 1`` per lane (``:504-519``), every layer with
    ``prefill=True``, logits of the last token of each lane (``logits_idx``, ``:894``)
    or of every token with ``all_rows``.  ``caches`` are updated in place."""
    q_batch, pos, cu = [], [], [0]
    for i, (n0, n1) in enumerate(seq_info):
        q_batch += [i] * n1
        pos += list(range(n0, n0 + n1))
        cu.append(cu[-1] + n1)
    q_batch = torch.tensor(q_batch, dtype=torch.int32)
    pos = torch.tensor(pos, dtype=torch.int32)
    cu = torch.tensor(cu, dtype=torch.int32)
    seqused = torch.tensor([n0 + n1 for n0, n1 in seq_info], dtype=torch.int32)
    t = token_values.shape[0]
    h = F.embedding(token_values.long(), weights["tok_embeddings"])
    for i, layer in enumerate(weights["layers"]):
        x = ref_rmsnorm(h, layer["attention_norm"], eps)
        xq = F.linear(x, layer["wq"]).view(t, n_heads, head_dim)
        xk = F.linear(x, layer["wk"]).view(t, n_kv_heads, head_dim)
        xv = F.linear(x, layer["wv"]).view(t, n_kv_heads, head_dim)
        attn = ref_gqa_attention_layer(xq, xk, xv, caches[i], pos, q_batch, None, freqs, cu,
                                       seqused, block_tbl, page_size, layer["window_left"])
        h = h + F.linear(attn.flatten(1, 2), layer["wo"])
        x = ref_rmsnorm(h, layer["ffn_norm"], eps)
        x1, x3 = F.linear(x, layer["w13"]).chunk(2, dim=1)
        h = h + F.linear(F.silu(x1) * x3, layer["w2"])
    h = ref_rmsnorm(h, weights["norm"], eps)
    if not all_rows:
        h = h[(cu[1:] - 1).long()]
    return F.linear(h, weights["output"])
