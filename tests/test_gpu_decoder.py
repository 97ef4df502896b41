"""The sharded decoder's decode step (world size 1, small shapes) against the CPU
fp32 restatement with the same weights, eagerly and replayed from a CUDA graph."""

from __future__ import annotations

import pytest
import torch

from oracle.ref_decoder import ref_decode_step, ref_prefill

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


def _weights_fp32(model):
    layers = []
    for layer in model.layers:
        d = {k: (v.float().cpu() if torch.is_tensor(v) else v) for k, v in layer.items()}
        d["wq"], d["wk"], d["wv"] = (w.float().cpu() for w in model.split_qkv(layer))
        layers.append(d)
    return {
        "layers": layers,
        "tok_embeddings": model.tok_embeddings.float().cpu(),
        "output": model.output.float().cpu(),
        "norm": model.norm.float().cpu(),
    }


def test_decode_steps_match_cpu_restatement(lib):
    from cwm_b200.decoder import DecoderArgs, DecodeState, ShardedDecoder

    args = DecoderArgs(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=512,
                       vocab_size=1024, local_window=64, page_size=256)
    model = ShardedDecoder(args, 0, 1, DEV, seed=3, std=0.05)
    assert [l["window_left"] for l in model.layers] == [-1, 63, 63, -1]
    bs, cols = 5, 3
    g = torch.Generator().manual_seed(11)
    table = torch.randperm(bs * cols, generator=g).reshape(bs, cols).to(torch.int32)
    cache = model.build_cache(bs * cols * args.page_size)
    for c in cache.caches:
        c.copy_((torch.randn(c.shape, generator=g) * 0.5).to(torch.bfloat16))
    ref_caches = [c.float().cpu() for c in cache.caches]
    weights = _weights_fp32(model)
    freqs = model.freqs.cpu()

    state = DecodeState(bs, table.to(DEV), args.page_size, DEV)
    seqlen = torch.tensor([100, 1, 300, 257, 64], dtype=torch.int32)
    tokens = torch.randint(0, args.vocab_size, (bs,), generator=g, dtype=torch.int32)
    state.copy_inputs(state.blktbl, tokens.to(DEV), seqlen.to(DEV))
    # eager warm-up step, checked
    logits = model.decode(state, cache).cpu()
    want = ref_decode_step(weights, tokens, seqlen, table, ref_caches, freqs, 4, 2, 128,
                           args.page_size, args.norm_eps)
    scale = want.abs().max().item()
    assert (logits - want).abs().max().item() <= 3e-2 * scale

    # captured step, replayed with new tokens and lengths (padded lanes at the end)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model.decode(state, cache)
    for step in range(3):
        seqlen = seqlen + 1
        nactive = bs - step
        seqlen[nactive:] = 0
        tokens = torch.randint(0, args.vocab_size, (bs,), generator=g, dtype=torch.int32)
        state.copy_inputs(state.blktbl, tokens.to(DEV), seqlen.to(DEV))
        state.set_actual_batch_size(nactive)
        graph.replay()
        torch.cuda.synchronize()
        want = ref_decode_step(weights, tokens, seqlen, table, ref_caches, freqs, 4, 2, 128,
                               args.page_size, args.norm_eps, nactive)
        got = out.cpu()
        assert (got[:nactive] - want[:nactive]).abs().max().item() <= 3e-2 * scale


def _small_model(seed=3):
    from cwm_b200.decoder import DecoderArgs, ShardedDecoder

    args = DecoderArgs(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=512,
                       vocab_size=1024, local_window=64, page_size=256)
    return args, ShardedDecoder(args, 0, 1, DEV, seed=seed, std=0.05)


def test_prefill_in_two_chunks_then_decode_matches_cpu_restatement(lib):
    """The model-level prefill pass (positions, logits of the last token only, cached
    prefixes) followed by decode steps: a prompt batch is prefilled in two calls cut
    by the engine's chunk splitter, then three tokens are decoded, and every set of
    logits is compared with the CPU restatement running the same chain on its own
    copy of the cache.  This drives the tensor-core prefill kernel from the model."""
    from cwm_b200.decoder import DecodeState
    from cwm_b200.layer import prefill_chunks

    args, model = _small_model()
    g = torch.Generator().manual_seed(21)
    prompts = [300, 70, 190]
    bs, cols = len(prompts), 3
    table = torch.randperm(bs * cols, generator=g).reshape(bs, cols).to(torch.int32)
    cache = model.build_cache(bs * cols * args.page_size)
    ref_caches = [c.float().cpu() for c in cache.caches]
    weights, freqs = _weights_fp32(model), model.freqs.cpu()
    toks = torch.randint(0, args.vocab_size, (sum(prompts),), generator=g, dtype=torch.int32)
    table_d = table.to(DEV)

    calls = prefill_chunks([(0, n) for n in prompts], 256)
    assert len(calls) == 3
    got_last, want_last = {}, {}
    for first_tok, last_tok, first_lane, lanes in calls:
        lane_tbl = table_d[first_lane : first_lane + len(lanes)]
        logits, _ = model.prefill(toks[first_tok:last_tok].to(DEV), lanes, lane_tbl, cache)
        want = ref_prefill(weights, toks[first_tok:last_tok], lanes,
                           table[first_lane : first_lane + len(lanes)], ref_caches, freqs, 4, 2,
                           128, args.page_size, args.norm_eps)
        scale = want.abs().max().item()
        assert logits.shape == want.shape
        assert (logits.cpu() - want).abs().max().item() <= 3e-2 * scale
        for i in range(len(lanes)):
            got_last[first_lane + i], want_last[first_lane + i] = logits[i].cpu(), want[i]
    # with logprobs every row is computed; the last-token rows must agree with the
    # rows the default path kept, and the log-probabilities with the restatement's
    lanes = [(0, 70)]
    cache2 = model.build_cache(bs * cols * args.page_size)
    sl = slice(300, 370)
    logits_lp, lps = model.prefill(toks[sl].to(DEV), lanes, table_d[1:2], cache2, logprobs=True)
    all_rows = ref_prefill(weights, toks[sl], lanes, table[1:2],
                           [torch.zeros_like(c) for c in ref_caches], freqs, 4, 2, 128,
                           args.page_size, args.norm_eps, all_rows=True)
    want_lp = -torch.nn.functional.cross_entropy(all_rows[:-1], toks[sl][1:].long(),
                                                 reduction="none")
    assert len(lps) == 1 and len(lps[0]) == 69
    assert (torch.tensor(lps[0]) - want_lp).abs().max().item() <= 5e-2
    assert (logits_lp[0].cpu() - all_rows[-1]).abs().max().item() <= 3e-2 * all_rows.abs().max().item()

    # decode three tokens on top of the prefilled cache
    state = DecodeState(bs, table_d, args.page_size, DEV)
    seqlen = torch.tensor([n + 1 for n in prompts], dtype=torch.int32)
    for _ in range(3):
        tokens = torch.randint(0, args.vocab_size, (bs,), generator=g, dtype=torch.int32)
        state.copy_inputs(state.blktbl, tokens.to(DEV), seqlen.to(DEV))
        logits = model.decode(state, cache).cpu()
        want = ref_decode_step(weights, tokens, seqlen, table, ref_caches, freqs, 4, 2, 128,
                               args.page_size, args.norm_eps)
        assert (logits - want).abs().max().item() <= 3e-2 * want.abs().max().item()
        seqlen = seqlen + 1


def test_graph_buckets_give_the_same_logits_as_a_tight_batch(lib):
    """Decode graphs per batch-size bucket in one pool: a live batch smaller than its
    bucket (padded lanes carry seqlen 0) gives the logits of an eager step over
    exactly the live lanes, and the bucket is the smallest that fits."""
    from cwm_b200.decoder import DecodeState, GraphedDecoder

    args, model = _small_model(seed=4)
    g = torch.Generator().manual_seed(31)
    max_batch, cols = 9, 2
    table = torch.randperm(max_batch * cols, generator=g).reshape(max_batch, cols).to(torch.int32).to(DEV)
    cache = model.build_cache(max_batch * cols * args.page_size)
    for c in cache.caches:
        c.copy_((torch.randn(c.shape, generator=g) * 0.5).to(torch.bfloat16))
    tokens = torch.randint(0, args.vocab_size, (max_batch,), generator=g, dtype=torch.int32).to(DEV)
    seqlen = torch.zeros(max_batch, dtype=torch.int32, device=DEV)
    gd = GraphedDecoder(model, cache, tokens, table, max_batch, num_graphs=4)
    assert gd.batch_sizes == [1, 4, 6, 9] and len(gd.graphs) == 4
    snapshot = [c.clone() for c in cache.caches]
    for nactive in (1, 3, 4, 5, 9):
        lens = torch.randint(1, cols * args.page_size - 4, (nactive,), generator=g,
                             dtype=torch.int32)
        seqlen.zero_()
        seqlen[:nactive] = lens.to(DEV)
        for c, s0 in zip(cache.caches, snapshot):
            c.copy_(s0)
        dg, logits = gd.step(table, tokens, seqlen, nactive)
        assert dg.state.batch_size == min(b for b in gd.batch_sizes if b >= nactive)
        got = logits.clone()
        torch.cuda.synchronize()
        # eager step over exactly the live lanes, on the same starting cache
        for c, s0 in zip(cache.caches, snapshot):
            c.copy_(s0)
        tight = DecodeState(nactive, table, args.page_size, DEV)
        tight.copy_inputs(tight.blktbl, tokens, seqlen)
        want = model.decode(tight, cache)
        # the attention kernels see the same tiles either way; the library GEMMs may
        # pick another algorithm for another row count, hence a tolerance
        assert (got - want).abs().max().item() <= 1e-2 * want.abs().max().item()
