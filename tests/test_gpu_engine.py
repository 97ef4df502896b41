"""Host KV offload and the generation engine on the GPU: the block-copy kernel
between pinned host memory and the device cache, the page-out / page-in round trip
of ``DynCache`` with its stream and event ordering, and whole requests through
``Engine.generate`` (chunked prefill with the prefix cache, graph-replayed decode
rounds, sampling) checked against the CPU restatement of the decoder."""

from __future__ import annotations

import queue

import pytest
import torch

from oracle.ref_decoder import ref_decode_step, ref_prefill

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def test_block_copy_between_pinned_host_and_device(lib):
    g = torch.Generator().manual_seed(1)
    rows, width, n_blocks = 16, 96, 5  # 192-byte rows in a 256-byte pitch on the device
    dev = torch.zeros(40 * rows, 128, dtype=torch.bfloat16, device=DEV)[:, :width]
    host = [torch.randn(rows, width, generator=g).to(torch.bfloat16).pin_memory()
            for _ in range(n_blocks)]
    blocks = [7, 0, 33, 12, 5]
    row_bytes = dev.stride(0) * 2
    dst = torch.tensor([dev.data_ptr() + b * rows * row_bytes for b in blocks], dtype=torch.int64,
                       device=DEV)
    src = torch.tensor([h.data_ptr() for h in host], dtype=torch.int64, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.cwm_block_copy(dst.data_ptr(), src.data_ptr(), n_blocks, rows, width * 2, row_bytes,
                            width * 2, stream)
    assert rc == 0, lib.cwm_last_error()
    torch.cuda.synchronize()
    for b, h in zip(blocks, host):
        assert torch.equal(dev[b * rows : (b + 1) * rows].cpu().view(torch.int16), h.view(torch.int16))
    assert dev[rows : 5 * rows].abs().sum().item() == 0  # blocks 1..4 untouched
    # and back into fresh host blocks
    back = [torch.zeros(rows, width, dtype=torch.bfloat16).pin_memory() for _ in range(n_blocks)]
    dst2 = torch.tensor([h.data_ptr() for h in back], dtype=torch.int64, device=DEV)
    rc = lib.cwm_block_copy(dst2.data_ptr(), dst.data_ptr(), n_blocks, rows, width * 2, width * 2,
                            row_bytes, stream)
    assert rc == 0, lib.cwm_last_error()
    torch.cuda.synchronize()
    for h, h2 in zip(host, back):
        assert torch.equal(h.view(torch.int16), h2.view(torch.int16))


def test_page_out_then_page_in_round_trip_is_bit_exact(lib):
    from cwm_b200.cache import RawCache
    from cwm_b200.hostcache import Cache, DynCache, DynCacheLane

    n_layers, hkv, d, page = 3, 2, 128, 256
    gpu = RawCache.build_dims(n_layers, hkv, d, 12 * page, DEV, torch.bfloat16)
    host = Cache(limit_toks=16 * page, node_len=page, page_len=page)
    host.preallocate(gpu)
    g = torch.Generator(device=DEV).manual_seed(2)
    lanes_blocks = [[3, 9, 1], [7, 4]]
    lanes = [DynCacheLane(blocks, [host.free_caches.pop() for _ in blocks], 0)
             for blocks in lanes_blocks]
    dyn = DynCache(gpu_cache=gpu, host_cache=host, cache_lanes=lanes)
    dyn.disable("page_in")
    want = []
    for n in range(n_layers):
        # the layer's rows are written on the compute stream right before the page-out,
        # which must wait for them (event ordering, no host sync in between)
        big = torch.randn(4096, 4096, device=DEV)
        (big @ big).sum()
        gpu.caches[n].copy_(torch.randn(gpu.caches[n].shape, generator=g, device=DEV))
        dyn.page_out(n)
        want.append(gpu.caches[n].clone())
    ready = dyn.host_cache_ready()
    ready.synchronize()
    for lane in lanes:
        for blk, hc in zip(lane.gpu_blocks, lane.cpu_blocks):
            for n in range(n_layers):
                assert torch.equal(hc._cache(n).view(torch.int16),
                                   want[n][blk * page : (blk + 1) * page].cpu().view(torch.int16))
    gpu.clear()
    lanes_in = [DynCacheLane(l.gpu_blocks, l.cpu_blocks, len(l.cpu_blocks)) for l in lanes]
    dyn_in = DynCache(gpu_cache=gpu, host_cache=host, cache_lanes=lanes_in)
    dyn_in.disable("page_out")
    with pytest.raises(AssertionError):
        dyn_in.cache_kv(0)  # no page-in was requested for the layer
    dyn_in.page_in(0)
    for n in range(n_layers):
        if n + 1 < n_layers:
            dyn_in.page_in(n + 1)  # the next layer's copy overlaps this layer's use
        k, v = dyn_in.cache_kv(n)  # waits for the layer's event on the current stream
        got = torch.cat([k, v], dim=1).clone()
        torch.cuda.synchronize()
        used = sorted(b for bl in lanes_blocks for b in bl)
        for blk in range(12):
            rows = slice(blk * page, (blk + 1) * page)
            if blk in used:
                assert torch.equal(got[rows].view(torch.int16), want[n][rows].view(torch.int16))
            else:
                assert got[rows].abs().sum().item() == 0


def _engine(model, **kw):
    from cwm_b200.engine import Engine, GenArgs

    args = GenArgs(max_batch=4, max_seq=16 * 256, cache_block=256, max_prefill=300,
                   min_prefill=0, min_prefill_batch=1, num_cuda_graphs=3, sync_freq=4,
                   host_cache_gb=0.05, **kw)
    return Engine(args, model, stop_tokens=[])


def _weights(model):
    from tests.test_gpu_decoder import _weights_fp32

    return _weights_fp32(model)


def _near_argmax(logits: torch.Tensor, token: int) -> bool:
    scale = logits.abs().max().item()
    return (logits.max() - logits[token]).item() <= 3e-2 * scale


def test_greedy_requests_follow_the_cpu_restatement(lib):
    """Requests of different lengths (one longer than max_prefill, one arriving later
    with a prompt prefix that is in the host cache by then) generate ``max_gen``
    tokens; every token the engine emitted must be an arg-max of the CPU restatement's
    logits along the engine's own sequence, within the bf16 tolerance."""
    from tests.test_gpu_decoder import _small_model
    from cwm_b200.engine import Packet

    args, model = _small_model(seed=6)
    eng = _engine(model, use_sampling=False, max_gen=6)
    g = torch.Generator().manual_seed(41)
    base = torch.randint(0, args.vocab_size, (700,), generator=g).tolist()
    prompts = {"a": base[:300], "b": base[300:370], "c": base[100:620]}
    q = queue.Queue()
    for k, v in prompts.items():
        q.put(Packet(thread_id=k, tokens=v))
    answers = {}
    gen = eng.generate(q)
    for pkt in gen:
        answers[pkt.thread_id] = pkt.tokens
        if len(answers) == 3:
            # a fourth request that shares the first 512 tokens of "c" (two cache pages)
            prompts["d"] = prompts["c"][:512] + base[650:690]
            q.put(Packet(thread_id="d", tokens=prompts["d"]))
            q.put(None)
    assert set(answers) == {"a", "b", "c", "d"}
    assert all(len(t) == 6 for t in answers.values())
    assert eng.host_cache.num_nodes >= 3  # pages of "a" and "c" were stored
    assert len(eng.table.free_blocks) == eng.table.nblocks and eng.table.nactive == 0

    weights, freqs = _weights(model), model.freqs.cpu()
    for k, prompt in prompts.items():
        cols = (len(prompt) + 8 + 255) // 256
        table = torch.arange(cols, dtype=torch.int32)[None]
        caches = [torch.zeros(cols * 256, 2 * 2 * 128) for _ in range(args.n_layers)]
        logits = ref_prefill(weights, torch.tensor(prompt, dtype=torch.int32), [(0, len(prompt))],
                             table, caches, freqs, 4, 2, 128, 256, args.norm_eps)[0]
        seqlen = len(prompt)
        for tok in answers[k]:
            assert _near_argmax(logits, tok), (k, tok, int(logits.argmax()))
            seqlen += 1
            logits = ref_decode_step(weights, torch.tensor([tok], dtype=torch.int32),
                                     torch.tensor([seqlen], dtype=torch.int32), table, caches,
                                     freqs, 4, 2, 128, 256, args.norm_eps)[0]


def test_sampled_requests_are_repeatable_and_respect_limits(lib):
    from tests.test_gpu_decoder import _small_model
    from cwm_b200.engine import Packet

    args, model = _small_model(seed=7)
    g = torch.Generator().manual_seed(43)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (40, 260, 90, 33, 150)]

    def run(seed):
        eng = _engine(model, use_sampling=True, temperature=0.8, logprobs=True, seed=seed)
        q = queue.Queue()
        for i, p in enumerate(prompts):
            q.put(Packet(thread_id=i, tokens=p, max_gen=3 + 2 * i,
                         top_p=0.9 if i % 2 else None))
        q.put(None)
        return {p.thread_id: p for p in eng.generate(q)}

    first, second, other = run(5), run(5), run(6)
    assert set(first) == set(range(5))
    for i in range(5):
        assert len(first[i].tokens) == 3 + 2 * i
        assert all(0 <= t < args.vocab_size for t in first[i].tokens)
        assert first[i].tokens == second[i].tokens  # same seed, same tokens
        assert len(first[i].logprobs) == len(first[i].tokens)
        assert len(first[i].sample_logprobs) == len(first[i].tokens)
        assert all(lp <= 0 for lp in first[i].logprobs)
    assert any(first[i].tokens != other[i].tokens for i in range(5))
