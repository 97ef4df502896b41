"""CPU fp32 restatement of a decode step of the GQA decoder.  TEST INFRASTRUCTURE
ONLY.  Follows the GQA path of ``cwm/fastgen/forward.py:467-821`` for an unsharded
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
