"""The sharded decoder's decode step (world size 1, small shapes) against the CPU
fp32 restatement with the same weights, eagerly and replayed from a CUDA graph."""

from __future__ import annotations

import pytest
import torch

from oracle.ref_decoder import ref_decode_step

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


def _weights_fp32(model):
    layers = []
    for layer in model.layers:
        layers.append({k: (v.float().cpu() if torch.is_tensor(v) else v) for k, v in layer.items()})
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
