"""Continuous-batching generation loop over the B200 attention path: lanes, the
KV-block allocator, chunked prefill, graph-replayed decode and sampling.

A restatement of the scheduling half of ``FastGen`` (``cwm/fastgen/generate.py``)
around this package's decoder: the same lane bookkeeping (``Lane``, ``:74-129``),
block accounting before every decode round (``_prepare_lanes``, ``:530-580``),
admission of queued and parked requests (``_add_lanes``, ``:582-654``), lane
retirement (``_kill_lane``, ``:1016-1057``), prompt processing with the host prefix
cache and the split into ``max_prefill``-token calls (``_prefill``, ``:819-994``),
``sync_freq`` decode steps per round replayed from the batch-size bucket's CUDA
graph (``_decode``, ``:729-817``), and sampling (``_sample``, ``:996-1014``).
Tokenizer, profiling and metrics hooks of the reference are left to the caller; a
``detokenize`` callable enables ``stop_str``.

``LaneTable`` holds everything that does not need a model (it works on CPU tensors
too, which is how its rules are tested); ``Engine`` adds the model calls.
"""

from __future__ import annotations

import bisect
import queue
from collections import deque
from collections.abc import Callable, Generator
from dataclasses import dataclass, field
from typing import Any

import torch
from torch.nn.functional import cross_entropy

from .hostcache import Cache, DynCache, DynCacheLane, hashints
from .iset import ISet


@dataclass
class Packet:
    """A request (``tokens`` = prompt) or an answer (``tokens`` = generation);
    ``cwm/fastgen/api.py:11-37``."""

    thread_id: Any
    tokens: list[int] = field(default_factory=list)
    text: str | None = None
    temperature: float | None = None
    top_p: float | None = None
    stop_str: str | None = None
    logprobs: list[float] | None = None
    sample_logprobs: list[float] | None = None
    max_gen: int | None = None


@dataclass
class GenArgs:
    """Engine settings; names and defaults of ``generate.py:37-69`` as far as they
    apply (``max_seq`` = KV-token budget, required here)."""

    use_sampling: bool = True
    temperature: float = 0.7
    top_p: float = 1.0
    logprobs: bool = False
    prompt_logprobs: bool = False
    max_batch: int = 128
    max_seq: int = -1
    max_gen: int | None = None
    host_cache_gb: float = 0
    num_cuda_graphs: int = 16
    cache_block: int = 256
    max_prefill: int = 4096
    min_prefill: int = 512
    min_prefill_batch: int = 8
    sync_freq: int = 10
    handover_frequency: int = 0
    seed: int = 0
    use_graphs: bool = True


@dataclass
class Lane(Packet):
    maxlen: int = 0
    prompt: list[int] = field(default_factory=list)
    blocks: list[int] = field(default_factory=list)
    blockset: ISet = field(default_factory=ISet)

    @staticmethod
    def from_pkt(p: Packet, max_seq: int, max_gen: int | None) -> "Lane":
        max_gen = p.max_gen if p.max_gen is not None else max_gen
        maxlen = max_seq if max_gen is None else min(len(p.tokens) + max_gen, max_seq)
        return Lane(thread_id=p.thread_id, temperature=p.temperature, top_p=p.top_p,
                    max_gen=max_gen, prompt=p.tokens, maxlen=maxlen, stop_str=p.stop_str)

    def all_tokens(self) -> list[int]:
        return self.prompt + self.tokens

    def add_block(self, bid: int) -> None:
        self.blockset.add(bid)
        self.blocks.append(bid)

    def free(self, free_set: ISet) -> None:
        free_set |= self.blockset
        self.blockset.clear()
        self.blocks = []

    def set_blocks(self, bset: ISet) -> None:
        assert not self.blockset
        self.blockset = bset
        self.blocks = bset.tolist()

    def __len__(self) -> int:
        return len(self.prompt) + len(self.tokens)


class LaneTable:
    """Lanes, their blocks and the per-lane device tensors of the engine."""

    def __init__(self, max_batch: int, max_seq: int, page_len: int, vocab_size: int,
                 device: torch.device | str) -> None:
        if max_seq <= 0 or max_seq % page_len or max_seq < max_batch * page_len:
            raise ValueError("max_seq must be a positive multiple of the page length and hold "
                             "one page per lane")
        self.max_batch, self.max_seq, self.page_len = max_batch, max_seq, page_len
        self.device = device
        self.nblocks = max_seq // page_len
        self.free_blocks = ISet.interval(0, self.nblocks)
        self.nactive = 0
        self.lane = [Lane("dead") for _ in range(max_batch)]
        self.parking: deque[Lane] = deque()
        self.top_p_lanes: set[int] = set()
        self.tokens = torch.randint(0, vocab_size, (max_batch,), dtype=torch.int, device=device)
        self.seqlen = torch.zeros(max_batch, dtype=torch.int, device=device)
        self.maxlen = torch.zeros(max_batch, dtype=torch.int, device=device)
        self.temps = torch.zeros(max_batch, dtype=torch.float, device=device)
        self.top_ps = torch.zeros(max_batch, dtype=torch.float, device=device)
        self.blktbl = torch.zeros((max_batch, self.nblocks), dtype=torch.int, device=device)

    def prepare_lanes(self, sync_freq: int) -> None:
        """Give every active lane room for ``sync_freq`` more tokens; when the free
        list runs dry, park the shortest lanes (they are re-admitted later and their
        prompt plus what they generated is prefilled again)."""
        page = self.page_len
        order = [i for _, i in sorted((-len(ln), i) for i, ln in enumerate(self.lane[: self.nactive]))]
        idx = 0
        while idx < self.nactive:
            lane = self.lane[order[idx]]
            if len(lane) + sync_freq <= len(lane.blocks) * page:
                idx += 1
                continue
            if not self.free_blocks:
                last = self.nactive - 1
                if last > 0:
                    self.kill_lane(order[last], park=True)
                    if idx == last:
                        break
                    # the lane that sat in slot `last` moved into the freed slot
                    for nxt in range(idx, last):
                        if order[nxt] == last:
                            order[nxt] = order[last]
                            break
            if self.free_blocks:
                bid = self.free_blocks.popleft()
                self.blktbl[order[idx], len(lane.blocks)] = bid
                lane.add_block(bid)
            else:
                # a single lane that owns every block: it reaches max_seq shortly
                assert self.nactive == 1
                idx = self.nactive
            assert min(self.max_seq, len(lane) + sync_freq) <= len(lane.blocks) * page

    def add_lanes(self, eoq: bool, q: "queue.Queue[Packet | None]", max_gen: int | None,
                  min_prefill: int, min_prefill_batch: int) -> tuple[bool, int, int]:
        """Admit parked lanes first, then queued requests, while lanes and blocks
        last.  Returns (queue exhausted, lanes added, checksum of what was read from
        the queue -- 0 when nothing was read)."""
        addend = 128 + self.page_len - 1  # head room of 128 tokens, rounded up to pages
        idx, tokens, cksum = self.nactive, 0, 0
        while idx < self.max_batch:
            lane: Lane | None = None
            parked = bool(self.parking)
            if parked:
                lane = self.parking.popleft()
            elif not eoq:
                try:
                    pkt = q.get(block=(idx == 0))
                except queue.Empty:
                    break
                if pkt is None:
                    eoq = True
                    cksum = hashints([cksum, 0])
                else:
                    cksum = hashints([cksum, hashints(pkt.tokens)])
                    lane = Lane.from_pkt(pkt, self.max_seq, max_gen)
            if lane is None:
                break
            ask = (len(lane) + addend) // self.page_len
            if ask > len(self.free_blocks):
                if parked:
                    self.parking.appendleft(lane)
                else:
                    self.parking.append(lane)
                break
            blocks, self.free_blocks = self.free_blocks.take(ask)
            lane.set_blocks(blocks)
            self.lane[idx] = lane
            tokens += len(lane)
            idx += 1
        if (tokens < min_prefill and idx - self.nactive < min_prefill_batch
                and not eoq and self.nactive > 0):
            # too little to be worth a prefill call while decoding has work: wait
            while idx > self.nactive:
                idx -= 1
                lane = self.lane[idx]
                lane.free(self.free_blocks)
                self.parking.appendleft(lane)
                self.lane[idx] = Lane("dead")
        return eoq, idx - self.nactive, cksum

    def kill_lane(self, lane: int, park: bool = False) -> None:
        """Retire an active lane; the last active lane takes its slot."""
        last = self.nactive - 1
        self.nactive = last
        self.lane[lane].free(self.free_blocks)
        if park:
            self.parking.append(self.lane[lane])
        per_lane = (self.seqlen, self.maxlen, self.temps, self.top_ps, self.blktbl)
        if lane != last:
            self.lane[lane] = self.lane[last]
            self.tokens[lane] = self.tokens[last]
            for t in per_lane:
                t[lane] = t[last]
            if last in self.top_p_lanes:
                self.top_p_lanes.remove(last)
                self.top_p_lanes.add(lane)
            else:
                self.top_p_lanes.discard(lane)
        else:
            self.top_p_lanes.discard(lane)
        self.lane[last] = Lane("dead")
        for t in per_lane:
            t[last] = 0


class Engine:
    """Generation engine around a ``ShardedDecoder`` (one tensor-parallel rank)."""

    def __init__(self, args: GenArgs, model, stop_tokens: list[int],
                 detokenize: Callable[[list[int]], str] | None = None,
                 group: "torch.distributed.ProcessGroup | None" = None) -> None:
        from .decoder import GraphedDecoder

        if args.max_seq <= 0:
            raise ValueError("GenArgs.max_seq (the KV-token budget) must be given")
        if args.sync_freq >= args.cache_block:
            raise ValueError("sync_freq must be smaller than the cache block")
        self.gen_args, self.model = args, model
        self.device = model.device
        self.group = group
        self.stop_tokens = list(stop_tokens)
        self.detokenize = detokenize
        self.page_len = self.block_len = args.cache_block
        self.max_batch, self.max_seq = args.max_batch, args.max_seq
        self.max_prefill = args.max_prefill
        self.min_prefill_batch = 1 if args.min_prefill_batch >= args.max_batch else args.min_prefill_batch
        self.gen_logprobs = args.logprobs or args.prompt_logprobs
        self.gen_prompt_logprobs = args.prompt_logprobs
        self.table = LaneTable(args.max_batch, args.max_seq, self.page_len,
                               model.args.vocab_size, self.device)
        self.cache = model.build_cache(self.table.nblocks * self.block_len)
        self.cache_ready: torch.cuda.Event | None = None
        self.host_cache = Cache(
            limit_toks=int(args.host_cache_gb * 1e9 / max(1, self.cache.bytes_per_token())),
            page_len=self.page_len, node_len=self.block_len)
        self.host_cache.preallocate(self.cache)
        # one generator per rank with the same seed: every rank draws the same uniforms
        self.rng = torch.Generator(device=self.device).manual_seed(args.seed)
        self.graphs = GraphedDecoder(model, self.cache, self.table.tokens, self.table.blktbl,
                                     args.max_batch, args.num_cuda_graphs, args.use_graphs)
        self.cache.clear()
        self.generating = False

    # ------------------------------------------------------------------ helpers
    def tensor(self, seq) -> torch.Tensor:
        return torch.tensor(seq, dtype=torch.int, device=self.device)

    def _check_consistent(self, val: int, what: str) -> None:
        """Every tensor-parallel rank must see the same value (an int32)."""
        if self.group is None:
            return
        t = self.tensor([val])
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN, group=self.group)
        if int(t[0]) != val:
            raise RuntimeError(f"Inconsistent {what} across mp ranks")

    def _sync_host_cache(self) -> None:
        if self.cache_ready is not None:
            self.cache_ready.wait()
            self.cache_ready = None

    def _sample(self, temps, top_ps, logits) -> tuple[torch.Tensor, torch.Tensor]:
        from .sampling import sample_logits

        return sample_logits(logits.contiguous(), temps.contiguous(),
                             top_ps.contiguous() if self.table.top_p_lanes else None,
                             self.gen_args.use_sampling, generator=self.rng)

    def _ended_lanes(self, tokens: torch.Tensor, toolong: torch.Tensor) -> list[int]:
        has_eos = torch.zeros_like(toolong)
        for st in self.stop_tokens:
            has_eos = torch.logical_or(has_eos, (tokens == st).sum(1))
        return (has_eos | toolong).tolist()

    def _has_stop_str(self, lane: Lane, n_new: int) -> bool:
        if lane.stop_str is None or self.detokenize is None:
            return False
        span = len(lane.stop_str) + n_new  # a stop string spans at most that many tokens
        return lane.stop_str in self.detokenize(lane.tokens[-span:])

    def _trim_packet(self, pkt: Lane) -> Packet:
        """Cut the answer after the first stop token (or stop string) and at
        ``max_gen``; decode rounds overshoot by up to ``sync_freq`` tokens."""
        trim = len(pkt.tokens)
        n = max(0, len(pkt.tokens) - self.gen_args.sync_freq - 1)
        for st in self.stop_tokens:
            if st in pkt.tokens[n:]:
                trim = min(trim, pkt.tokens.index(st, n) + 1)
        if pkt.max_gen is not None:
            trim = min(trim, pkt.max_gen)
        if pkt.stop_str is not None and self.detokenize is not None \
                and pkt.stop_str in self.detokenize(pkt.tokens[:trim]):
            lo, hi = 0, trim  # stop_str not in tokens[:lo], in tokens[:hi]
            while hi - lo > 1:
                mid = lo + (hi - lo) // 2
                if pkt.stop_str in self.detokenize(pkt.tokens[:mid]):
                    hi = mid
                else:
                    lo = mid
            trim = hi
        pkt.tokens = pkt.tokens[:trim]
        if pkt.sample_logprobs is not None:
            pkt.sample_logprobs = pkt.sample_logprobs[:trim]
        if pkt.logprobs is not None:
            keep = len(pkt.prompt) - 1 + trim if self.gen_prompt_logprobs else trim
            pkt.logprobs = pkt.logprobs[:keep]
        return pkt

    # ------------------------------------------------------------------- decode
    def _decode(self) -> tuple[torch.Tensor, list[list[float]], list[list[float]]]:
        """Up to ``sync_freq`` decode steps for the active lanes without a host
        sync in between; returns tokens ``(nactive, nsteps)`` and the two kinds of
        log-probabilities."""
        tb = self.table
        nactive = tb.nactive
        seqlen, blktbl, tokens = tb.seqlen, tb.blktbl, tb.tokens
        dg = self.graphs.bucket(nactive)
        maxsl = int(seqlen.max().item())
        assert maxsl < self.max_seq
        nsteps = min(self.max_seq - maxsl, self.gen_args.sync_freq)
        output = torch.empty((nactive, nsteps), dtype=torch.int, device=self.device)
        shape = (nactive, nsteps) if self.gen_logprobs else (0,)
        logprobs = torch.empty(shape, dtype=torch.float32, device=self.device)
        sample_logprobs = torch.empty(shape, dtype=torch.float32, device=self.device)
        dg.state.set_actual_batch_size(nactive)
        for i in range(nsteps):
            dg.state.copy_inputs(blktbl, tokens, seqlen)
            if dg.graph is not None:
                dg.graph.replay()
                logits = dg.logits
            else:
                logits = self.model.decode(dg.state, self.cache)
            logits = logits[:nactive]
            new_tokens, new_slp = self._sample(tb.temps[:nactive], tb.top_ps[:nactive], logits)
            output[:, i] = new_tokens
            if self.gen_logprobs:
                logprobs[:, i] = -cross_entropy(logits, new_tokens, reduction="none")
                sample_logprobs[:, i] = new_slp
            tokens, seqlen, blktbl = dg.state.tokens, dg.state.seqlen, dg.state.blktbl
            tokens[:nactive].copy_(new_tokens)
            seqlen[:nactive].add_(1)
        tb.tokens[:nactive].copy_(tokens[:nactive])
        tb.seqlen[:nactive].copy_(seqlen[:nactive])
        return output, logprobs.tolist(), sample_logprobs.tolist()

    # ------------------------------------------------------------------ prefill
    def _prefill(self, nprefill: int):
        """Fill the KV cache of the ``nprefill`` lanes just added and draw their
        first token.  Returns (tokens, logprobs, sample_logprobs, toolong)."""
        tb = self.table
        first, new_nactive = tb.nactive, tb.nactive + nprefill
        host_cache, gpu_cache = self.host_cache, self.cache
        cache_lanes: list[DynCacheLane] = []
        seq_info: list[tuple[int, int]] = []
        start_pos: list[int] = []
        tokens_list: list[int] = []
        seqlen_list, maxlen_list, temps_list, top_ps_list = [], [], [], []
        for i in range(first, new_nactive):
            lane = tb.lane[i]
            toks = lane.all_tokens()
            assert toks and len(toks) < self.max_seq
            cache_lane = host_cache.prepare_lane(gpu_cache, lane.blocks, toks)
            cache_lanes.append(cache_lane)
            cached = host_cache.node_len * cache_lane.ready_count
            if cached == len(toks):
                cached -= 1  # never an empty sequence: the last token is processed again
            seq_info.append((cached, len(toks) - cached))
            start_pos.append(len(tokens_list))
            tokens_list.extend(toks[cached:])
            tb.blktbl[i, : len(lane.blocks)] = self.tensor(lane.blocks)
            seqlen_list.append(len(toks))
            maxlen_list.append(lane.maxlen)
            temps_list.append(lane.temperature if lane.temperature is not None
                              else self.gen_args.temperature)
            top_ps_list.append(lane.top_p if lane.top_p is not None else self.gen_args.top_p)
            if top_ps_list[-1] != 1:
                tb.top_p_lanes.add(i)
        dyn_cache = DynCache(gpu_cache=gpu_cache, host_cache=host_cache, cache_lanes=cache_lanes)

        # calls of at most max_prefill new tokens; a lane cut by a call continues in the next
        fst_tok, lst_tok, fst_idx = 0, self.max_prefill, 0
        blktbl = tb.blktbl[first:new_nactive]
        logits_list: list[torch.Tensor] = []
        logprobs: list[list[float]] = [[] for _ in start_pos] if self.gen_prompt_logprobs else []
        while lst_tok < len(tokens_list):
            lst_idx = bisect.bisect_left(start_pos, lst_tok, fst_idx)
            split_idx = lst_idx - 1
            cached, ntoks = seq_info[split_idx]
            new_ntoks = lst_tok - start_pos[split_idx]
            if new_ntoks == ntoks:  # keep the lane's last token for the next call
                new_ntoks -= 1
                lst_tok -= 1
            seq_info[split_idx] = (cached, new_ntoks)
            dyn_cache.disable("page_out")
            logits, lp_chunk = self.model.prefill(
                self.tensor(tokens_list[fst_tok:lst_tok]), seq_info[fst_idx:lst_idx],
                blktbl[fst_idx:lst_idx], dyn_cache, logprobs=self.gen_prompt_logprobs)
            if lp_chunk is not None:
                for i, lp in enumerate(lp_chunk):
                    logprobs[fst_idx + i].extend(lp)
                new_ntoks -= 1
                lst_tok -= 1
            dyn_cache.disable("page_in")
            logits_list.append(logits[:-1])
            seq_info[split_idx] = (cached + new_ntoks, ntoks - new_ntoks)
            start_pos[split_idx] += new_ntoks
            fst_idx, fst_tok = split_idx, lst_tok
            lst_tok += self.max_prefill
        dyn_cache.enable("page_out")
        logits, lp_chunk = self.model.prefill(
            self.tensor(tokens_list[fst_tok:]), seq_info[fst_idx:], blktbl[fst_idx:], dyn_cache,
            logprobs=self.gen_prompt_logprobs)
        if lp_chunk is not None:
            for i, lp in enumerate(lp_chunk):
                logprobs[fst_idx + i].extend(lp)
        logits_list.append(logits)
        logits = torch.cat(logits_list, dim=0)

        seqlen, maxlen = self.tensor(seqlen_list), self.tensor(maxlen_list)
        temps = torch.tensor(temps_list, dtype=torch.float, device=self.device)
        top_ps = torch.tensor(top_ps_list, dtype=torch.float, device=self.device)
        host_cache.tick()
        assert self.cache_ready is None
        self.cache_ready = dyn_cache.host_cache_ready()

        next_tokens, sample_lp = self._sample(temps, top_ps, logits)
        if self.gen_logprobs:
            token_lp = (-cross_entropy(logits, next_tokens, reduction="none"))[:, None].tolist()
            if self.gen_prompt_logprobs:
                for i, lp in enumerate(token_lp):
                    logprobs[i].extend(lp)
            else:
                logprobs = token_lp
            sample_logprobs = sample_lp[:, None].tolist()
        else:
            sample_logprobs = []
        sl = slice(first, new_nactive)
        tb.tokens[sl] = next_tokens
        tb.seqlen[sl] = seqlen + 1
        tb.maxlen[sl] = maxlen
        tb.temps[sl] = temps
        tb.top_ps[sl] = top_ps
        tb.nactive = new_nactive
        return next_tokens[:, None], logprobs, sample_logprobs, (seqlen + 1) >= maxlen

    # --------------------------------------------------------------------- loop
    def generate(self, q: "queue.Queue[Packet | None]") -> Generator[Packet | None, None, None]:
        """Serve the requests put on ``q`` (``None`` ends the stream); yields one
        ``Packet`` per request, in completion order."""
        assert not self.generating, "multiple generators cannot run concurrently"
        self.generating = True
        try:
            yield from self._generate(q)
        finally:
            self.generating = False

    @torch.inference_mode()
    def _generate(self, q) -> Generator[Packet | None, None, None]:
        tb = self.table
        eoq, num_iters = False, 0
        while not eoq or tb.parking or tb.nactive > 0:
            if self.gen_args.handover_frequency > 0:
                num_iters += 1
                if num_iters == self.gen_args.handover_frequency:
                    num_iters = 0
                    yield None
            done: list[int] = []
            tokens_list: list[list[int]] = []
            logprobs_list: list = []
            sample_logprobs_list: list = []
            tb.prepare_lanes(self.gen_args.sync_freq)
            if tb.nactive > 0:
                tokens, logprobs, sample_logprobs = self._decode()
                toolong = (tb.seqlen >= tb.maxlen)[: tb.nactive]
                done += self._ended_lanes(tokens, toolong)
                tokens_list += tokens.tolist()
                logprobs_list += logprobs
                sample_logprobs_list += sample_logprobs
            self._sync_host_cache()
            self.host_cache.maintain()
            eoq, added, cksum = tb.add_lanes(eoq, q, self.gen_args.max_gen,
                                             self.gen_args.min_prefill, self.min_prefill_batch)
            if cksum:
                self._check_consistent(cksum, "input queue")
            if added:
                tokens, logprobs, sample_logprobs, toolong = self._prefill(added)
                done += self._ended_lanes(tokens, toolong)
                tokens_list += tokens.tolist()
                logprobs_list += logprobs
                sample_logprobs_list += sample_logprobs
            # in reverse, so that retiring a lane does not move one still to be visited
            for i in reversed(range(tb.nactive)):
                lane = tb.lane[i]
                lane.tokens += tokens_list[i]
                if self.gen_logprobs:
                    lane.logprobs = (lane.logprobs or []) + logprobs_list[i]
                    lane.sample_logprobs = (lane.sample_logprobs or []) + sample_logprobs_list[i]
                if done[i] or self._has_stop_str(lane, len(tokens_list[i])):
                    yield self._trim_packet(lane)
                    # retiring shuffles lanes: pending copies to host memory must land first
                    self._sync_host_cache()
                    tb.kill_lane(i)
