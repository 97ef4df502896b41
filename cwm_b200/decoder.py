"""GQA-only decode pass of a CWM-shaped decoder, tensor-parallel over KV heads.

A slim restatement of the decode path of ``cwm/fastgen/forward.py:467-821`` for the
model family CWM uses (grouped-query attention, SwiGLU, RMSNorm, rotary embedding,
interleaved local/global layers): the projections stay library GEMMs
(``F.linear``), the attention path runs on this package's kernels, and the two
row-parallel products of a layer are summed over the tensor-parallel group by
all-reduce (``forward.py:763-768,782-785``).  Embedding and output are
vocabulary-parallel (``forward.py:134-167,803-811``).  Weights are random
(there are no checkpoints here); it exists to measure whole-step decode
throughput with the attention kernels in place, inside a CUDA graph like the
reference's decode loop (``cwm/fastgen/generate.py:338-373,779-804``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .attn_bias import AttnBias
from .cache import RawCache
from .kernels import add_rmsnorm, rmsnorm
from .layer import gqa_attention, rope_freqs, window_size_left
from .tp import Collectives, HeadShard, shard_heads


@dataclass
class DecoderArgs:
    """Shapes of the decoder.  Defaults: CWM-32B."""

    dim: int = 6144
    n_layers: int = 64
    n_heads: int = 48
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 21504
    vocab_size: int = 128256
    rope_theta: float = 1e6
    norm_eps: float = 1e-5
    window_pattern: int = 4  # 3 local : 1 global
    local_window: int | None = 8192
    global_window: int | None = None
    global_last_layer: bool = True
    page_size: int = 256


class DecodeState:
    """Graph-stable inputs of a decode step (``ModelState``, ``forward.py:39-131``):
    tokens, per-lane key counts (which already include the token being fed), the
    block table and the live batch size, all device tensors updated in place."""

    def __init__(self, batch_size: int, block_tbl: torch.Tensor, page_size: int,
                 device: torch.device) -> None:
        self.batch_size = batch_size
        self.tokens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        capacity = block_tbl.shape[1] * page_size
        self.bias = AttnBias.from_seqlens([1] * batch_size, [capacity] * batch_size,
                                          block_tbl[:batch_size], page_size)
        self.actual_batch_size = torch.tensor(batch_size, dtype=torch.int64, device=device)

    @property
    def seqlen(self) -> torch.Tensor:
        return self.bias.k_seqinfo.seqlen

    @property
    def blktbl(self) -> torch.Tensor:
        return self.bias.block_tables

    def set_actual_batch_size(self, n: int) -> None:
        self.actual_batch_size.fill_(n)

    def copy_inputs(self, blktbl: torch.Tensor, tokens: torch.Tensor, seqlen: torch.Tensor) -> None:
        if blktbl.data_ptr() != self.blktbl.data_ptr():
            self.blktbl.copy_(blktbl[: self.batch_size])
        if tokens.data_ptr() != self.tokens.data_ptr():
            self.tokens.copy_(tokens[: self.batch_size])
        if seqlen.data_ptr() != self.seqlen.data_ptr():
            self.seqlen.copy_(seqlen[: self.batch_size])


class ShardedDecoder:
    """One tensor-parallel rank of the decoder, with random bf16 weights."""

    def __init__(self, args: DecoderArgs, rank: int, world: int, device: torch.device,
                 dtype: torch.dtype = torch.bfloat16, seed: int = 0, std: float = 0.02,
                 group: dist.ProcessGroup | None = None, collectives: bool = True) -> None:
        """``collectives=False`` builds the shard of ``rank`` without a process group
        and skips the all-reduces and the logits gather: the per-GPU work of a
        ``world``-way run on a single GPU, for profiling."""
        if args.ffn_dim % world or args.vocab_size % world:
            raise ValueError("ffn_dim and vocab_size must be divisible by the group size")
        self.args = args
        self.rank, self.world = rank, world
        self.device, self.dtype = device, dtype
        self.shard: HeadShard = shard_heads(rank, world, args.n_heads, args.n_kv_heads)
        self.coll = Collectives(group) if world > 1 and collectives else None
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)

        def w(*shape: int) -> torch.Tensor:
            t = torch.empty(shape, device=device, dtype=dtype)
            return t.normal_(0.0, std, generator=gen)

        hq, hkv, d = self.shard.n_q, self.shard.n_kv, args.head_dim
        ffn = args.ffn_dim // world
        self.layers = []
        for i in range(args.n_layers):
            self.layers.append({
                "wq": w(hq * d, args.dim),
                "wk": w(hkv * d, args.dim),
                "wv": w(hkv * d, args.dim),
                "wo": w(args.dim, hq * d),
                "w13": w(2 * ffn, args.dim),
                "w2": w(args.dim, ffn),
                "attention_norm": torch.ones(args.dim, device=device, dtype=dtype),
                "ffn_norm": torch.ones(args.dim, device=device, dtype=dtype),
                "window_left": window_size_left(i, args.n_layers, args.window_pattern,
                                                args.local_window, args.global_window,
                                                args.global_last_layer),
            })
        self.norm = torch.ones(args.dim, device=device, dtype=dtype)
        self.tok_embeddings = w(args.vocab_size // world, args.dim)
        self.output = w(args.vocab_size // world, args.dim)
        self.freqs = rope_freqs(d, args.rope_theta).to(device)

    def build_cache(self, length: int) -> RawCache:
        return RawCache.build_dims(self.args.n_layers, self.shard.n_kv, self.args.head_dim, length,
                                   self.device, self.dtype)

    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.coll is None else self.coll.all_reduce(x)

    def _embed(self, tokens: torch.Tensor) -> torch.Tensor:
        """Vocabulary-parallel embedding, ``forward.py:134-167``."""
        local = self.tok_embeddings.shape[0]
        start = self.rank * local
        mask = (tokens < start) | (tokens >= start + local)
        idx = torch.where(mask, torch.zeros_like(tokens), tokens - start)
        h = F.embedding(idx, self.tok_embeddings)
        h = h.masked_fill(mask[:, None], 0.0)
        return self._all_reduce(h)

    @torch.inference_mode()
    def decode(self, state: DecodeState, cache: RawCache) -> torch.Tensor:
        """One decode step for every lane of ``state``; returns fp32 logits
        ``(batch, vocab)``.  Op order as in ``forward.py:563-821`` (GQA branch)."""
        a = self.args
        hq, hkv, d = self.shard.n_q, self.shard.n_kv, a.head_dim
        q_seqpos = state.seqlen - 1  # forward.py:525
        h = self._embed(state.tokens)
        # every residual add is fused with the normalisation that follows it
        x = rmsnorm(h, self.layers[0]["attention_norm"], a.norm_eps)
        for i, layer in enumerate(self.layers):
            xq = F.linear(x, layer["wq"]).view(-1, hq, d)
            xk = F.linear(x, layer["wk"]).view(-1, hkv, d)
            xv = F.linear(x, layer["wv"]).view(-1, hkv, d)
            attn = gqa_attention(xq, xk, xv, cache, i, state.bias, q_seqpos, None,
                                 state.actual_batch_size, self.freqs, layer["window_left"])
            h_out = self._all_reduce(F.linear(attn.flatten(1, 2), layer["wo"]))
            x = add_rmsnorm(h, h_out, layer["ffn_norm"], a.norm_eps)
            x13 = F.linear(x, layer["w13"])
            x1, x3 = x13.chunk(2, dim=1)
            h_out = self._all_reduce(F.linear(F.silu(x1).mul_(x3), layer["w2"]))
            next_norm = (self.layers[i + 1]["attention_norm"] if i + 1 < len(self.layers)
                         else self.norm)
            x = add_rmsnorm(h, h_out, next_norm, a.norm_eps)
        h = x
        logits = F.linear(h, self.output)
        if self.coll is not None:
            gathered = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(gathered, logits, group=self.coll.group)
            logits = torch.cat(gathered, dim=-1)
        return logits.float()
