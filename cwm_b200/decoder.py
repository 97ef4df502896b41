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

from .attention import silu_mul
from .attn_bias import AttnBias
from .cache import ModelCache, RawCache
from .kernels import add_rmsnorm, rmsnorm
from .layer import gqa_attention_packed, prefill_positions, rope_freqs, window_size_left
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
                 device: torch.device, tokens: torch.Tensor | None = None) -> None:
        """``tokens`` (optional): the engine-wide token tensor, of which the state
        keeps the view ``tokens[:batch_size]`` like the reference; without it the
        state owns its tokens.  The block table is always a view of ``block_tbl``."""
        self.batch_size = batch_size
        self.tokens = (torch.zeros(batch_size, dtype=torch.int32, device=device)
                       if tokens is None else tokens[:batch_size])
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
    """One tensor-parallel rank of the decoder, with random bf16 weights.

    The q, k and v projections of a layer are one stacked weight ``wqkv`` (one
    product instead of three), and ``w13`` stacks the two input projections of the
    SwiGLU block."""

    def __init__(self, args: DecoderArgs, rank: int, world: int, device: torch.device,
                 dtype: torch.dtype = torch.bfloat16, seed: int = 0, std: float = 0.02,
                 group: dist.ProcessGroup | None = None, collectives: bool = True,
                 peer_all_reduce: bool = False, fuse_all_reduce: bool = True) -> None:
        """``collectives=False`` builds the shard of ``rank`` without a process group
        and skips the all-reduces and the logits gather: the per-GPU work of a
        ``world``-way run on a single GPU, for profiling.  ``peer_all_reduce`` sends
        the row-parallel sums through this package's peer-memory kernel instead of
        the process group's all-reduce (all ranks on one node); with it,
        ``fuse_all_reduce`` lets passes whose token count divides by the group size run
        each all-reduce, the residual add and the RMSNorm after it as one kernel."""
        if args.ffn_dim % world or args.vocab_size % world:
            raise ValueError("ffn_dim and vocab_size must be divisible by the group size")
        self.args = args
        self.rank, self.world = rank, world
        self.device, self.dtype = device, dtype
        self.shard: HeadShard = shard_heads(rank, world, args.n_heads, args.n_kv_heads)
        self.coll = None
        self.fuse_all_reduce = fuse_all_reduce
        if world > 1 and collectives:
            from .tp import PeerAllReduce

            peer = PeerAllReduce(group, device) if peer_all_reduce else None
            self.coll = Collectives(group, peer)
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)

        def w(*shape: int) -> torch.Tensor:
            t = torch.empty(shape, device=device, dtype=dtype)
            return t.normal_(0.0, std, generator=gen)

        hq, hkv, d = self.shard.n_q, self.shard.n_kv, args.head_dim
        ffn = args.ffn_dim // world
        self.layers = []
        for i in range(args.n_layers):
            self.layers.append({
                "wqkv": w((hq + 2 * hkv) * d, args.dim),
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

    def split_qkv(self, layer: dict) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Views ``(wq, wk, wv)`` of a layer's stacked projection weight."""
        hq, hkv, d = self.shard.n_q, self.shard.n_kv, self.args.head_dim
        return torch.split(layer["wqkv"], [hq * d, hkv * d, hkv * d], dim=0)

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
        h = self._all_reduce(h)
        # the peer kernel returns a view of a buffer that later calls reuse; the
        # residual stream lives for the whole pass, so it gets memory of its own
        return h.clone() if self.coll is not None and self.coll.peer is not None else h

    def _forward(self, tokens: torch.Tensor, bias: AttnBias, q_seqpos: torch.Tensor,
                 q_batch: torch.Tensor | None, actual_batch_size: torch.Tensor | None,
                 cache: ModelCache, logits_idx: torch.Tensor | None) -> torch.Tensor:
        """The GQA path of ``_forward`` (``forward.py:467-821``): embedding, the layers
        (with the page-in request for the next layer issued before each one,
        ``forward.py:561-568``), final norm, rows ``logits_idx`` only when given, the
        vocabulary-parallel output product and its gather.  fp32 logits."""
        a = self.args
        hq, hkv = self.shard.n_q, self.shard.n_kv
        cache.page_in(0)
        h = self._embed(tokens)
        # every residual add is fused with the normalisation that follows it, and with
        # the all-reduce before it when the peer-memory kernel serves this shape (one
        # choice for the whole pass: that kernel keeps only this rank's rows of h current)
        fused = (self.fuse_all_reduce and self.coll is not None
                 and self.coll.fuses_add_rmsnorm(h.shape[0], h.shape[1], h.dtype))
        x = rmsnorm(h, self.layers[0]["attention_norm"], a.norm_eps)
        n_layers = len(self.layers)
        for i, layer in enumerate(self.layers):
            if i + 1 < n_layers:
                cache.page_in(i + 1)
            qkv = F.linear(x, layer["wqkv"])
            attn = gqa_attention_packed(qkv, hq, hkv, cache, i, bias, q_seqpos, q_batch,
                                        actual_batch_size, self.freqs, layer["window_left"])
            next_norm = self.layers[i + 1]["attention_norm"] if i + 1 < n_layers else self.norm
            if self.coll is None:
                x = add_rmsnorm(h, F.linear(attn.flatten(1, 2), layer["wo"]), layer["ffn_norm"],
                                a.norm_eps)
                x = add_rmsnorm(h, F.linear(silu_mul(F.linear(x, layer["w13"])), layer["w2"]),
                                next_norm, a.norm_eps)
            else:
                x = self.coll.linear_all_reduce_add_rmsnorm(
                    attn.flatten(1, 2), layer["wo"], h, layer["ffn_norm"], a.norm_eps, fused)
                x = self.coll.linear_all_reduce_add_rmsnorm(
                    silu_mul(F.linear(x, layer["w13"])), layer["w2"], h, next_norm, a.norm_eps,
                    fused)
        if logits_idx is not None:
            x = x[logits_idx]
        logits = F.linear(x, self.output)
        if self.coll is not None:
            gathered = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(gathered, logits, group=self.coll.group)
            logits = torch.cat(gathered, dim=-1)
        return logits.float()

    @torch.inference_mode()
    def decode(self, state: DecodeState, cache: ModelCache) -> torch.Tensor:
        """One decode step for every lane of ``state`` (``decode``,
        ``forward.py:929-961``); returns fp32 logits ``(batch, vocab)``."""
        q_seqpos = state.seqlen - 1  # forward.py:525
        return self._forward(state.tokens, state.bias, q_seqpos, None, state.actual_batch_size,
                             cache, None)

    @torch.inference_mode()
    def prefill(self, token_values: torch.Tensor, seq_info: list[tuple[int, int]],
                block_tbl: torch.Tensor, cache: ModelCache, logprobs: bool = False
                ) -> tuple[torch.Tensor, list[list[float]] | None]:
        """Prompt processing (``prefill``, ``forward.py:824-926``).

        ``token_values``: int32, the new tokens of all lanes concatenated;
        ``seq_info``: per lane ``(cached, new)`` token counts; ``block_tbl``: the
        lanes' rows of the block table (a row slice is fine).  Fills the cache rows
        of the new tokens and returns the fp32 logits of the last token of each lane
        and, with ``logprobs``, the log-probabilities of the non-predicted tokens."""
        page = self.args.page_size
        q_seqlen = [n1 for _, n1 in seq_info]
        bias = AttnBias.from_seqlens(q_seqlen, [n0 + n1 for n0, n1 in seq_info], block_tbl, page)
        q_batch, q_seqpos = prefill_positions(seq_info, token_values.device)
        logits_idx = (bias.q_seqinfo.seqstart[1:] - 1).long()
        logits = self._forward(token_values, bias, q_seqpos, q_batch, None, cache,
                               None if logprobs else logits_idx)
        if not logprobs:
            return logits, None
        token_logprobs = (-F.cross_entropy(logits[:-1], token_values[1:].to(torch.int64),
                                           reduction="none")).tolist()
        seq_logprobs, beg = [], 0
        for sl in q_seqlen:
            seq_logprobs.append(token_logprobs[beg : beg + sl - 1])
            beg += sl
        return logits[logits_idx], seq_logprobs


@dataclass
class DecodeGraph:
    state: DecodeState
    graph: torch.cuda.CUDAGraph | None
    logits: torch.Tensor | None


class GraphedDecoder:
    """Decode steps replayed from CUDA graphs, one per batch-size bucket, all in one
    memory pool, as the reference engine builds them (``cwm/fastgen/generate.py:
    319-373``) and picks them (``:751-754``): the smallest bucket that holds the
    live lanes; lanes beyond them carry ``seqlen = 0``."""

    def __init__(self, model: ShardedDecoder, cache: ModelCache, tokens: torch.Tensor,
                 blktbl: torch.Tensor, max_batch: int, num_graphs: int = 16,
                 use_graphs: bool = True) -> None:
        self.model, self.cache = model, cache
        # bucket sizes: linspace(1, max_batch, num_graphs) rounded, duplicates dropped
        sizes = torch.linspace(1, max_batch, max(2, num_graphs), dtype=torch.float32)
        self.batch_sizes = sorted(set(sizes.round().int().tolist()))
        graphs: list[DecodeGraph] = []
        pool = None
        page = model.args.page_size
        for bs in reversed(self.batch_sizes):
            state = DecodeState(bs, blktbl, page, model.device, tokens)
            state.seqlen.zero_()  # every lane padded while capturing: the cache is not touched
            graph, logits = None, None
            if use_graphs:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    model.decode(state, cache)  # first launches outside the capture
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, pool=pool):
                    logits = model.decode(state, cache)
                if pool is None:
                    pool = graph.pool()
            graphs.append(DecodeGraph(state, graph, logits))
        self.graphs = list(reversed(graphs))

    def bucket(self, nactive: int) -> DecodeGraph:
        import bisect

        idx = bisect.bisect_left(self.batch_sizes, nactive)
        if idx >= len(self.graphs):
            raise ValueError(f"{nactive} live lanes exceed the largest bucket")
        return self.graphs[idx]

    @torch.inference_mode()
    def step(self, blktbl: torch.Tensor, tokens: torch.Tensor, seqlen: torch.Tensor,
             nactive: int) -> tuple[DecodeGraph, torch.Tensor]:
        """One decode step for the first ``nactive`` lanes of the engine-wide
        ``tokens`` / ``seqlen`` / ``blktbl`` tensors; returns the bucket used and
        the logits of the live lanes."""
        dg = self.bucket(nactive)
        dg.state.set_actual_batch_size(nactive)
        dg.state.copy_inputs(blktbl, tokens, seqlen)
        if dg.graph is not None:
            dg.graph.replay()
            logits = dg.logits
        else:
            logits = self.model.decode(dg.state, self.cache)
        return dg, logits[:nactive]
