"""The whole per-layer step on the GPU (rotary embedding + KV-cache write +
attention, cwm/fastgen/forward.py:608-656) against the CPU oracle, eagerly and
replayed from a CUDA graph with lengths that change between replays."""

from __future__ import annotations

import pytest
import torch

from oracle import ref_gqa_attention_layer, ref_rope_freqs

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
HQ, HKV, D, PAGE = 12, 2, 128, 256


@pytest.fixture(scope="module")
def ops(lib):
    import cwm_b200

    return cwm_b200


def _cache_checks(cache_gpu, ref_cache):
    got = cache_gpu.cpu()
    # V rows: bit-exact copies of the inputs; K rows: our rotation, within one rounding step
    assert torch.equal(got[:, HKV * D :].view(torch.int16), ref_cache[:, HKV * D :].view(torch.int16))
    assert (got[:, : HKV * D].float() - ref_cache[:, : HKV * D].float()).abs().max().item() <= 2e-2
    # rows that were not written are untouched, bit for bit
    untouched = (ref_cache == 0).all(dim=1)
    assert torch.equal(got[untouched].view(torch.int16), ref_cache[untouched].view(torch.int16))


@pytest.mark.parametrize("window_left", [-1, 8191, 100])
def test_prefill_then_decode_layer(ops, window_left):
    g = torch.Generator().manual_seed(window_left + 10)
    n_pages = 16
    table = torch.randperm(n_pages, generator=g).reshape(4, 4).to(torch.int32)
    freqs = ref_rope_freqs(D, 1e6)
    ref_cache = torch.zeros(n_pages * PAGE, 2 * HKV * D, dtype=torch.bfloat16)
    cache = ops.RawCache.build_dims(1, HKV, D, n_pages * PAGE, DEV, torch.bfloat16)

    # two prefill chunks per lane (the second with a cached prefix), then three decode steps
    lens = [0, 0, 0, 0]
    steps = [[300, 17, 0, 512], [211, 0, 130, 300], [1, 1, 1, 1], [1, 1, 1, 1], [1, 1, 1, 1]]
    for new in steps:
        lanes = [i for i, n in enumerate(new) if n > 0]
        seq_info = [(lens[i], new[i]) for i in lanes]
        decode = all(n == 1 for n in new)
        q_batch, q_pos = ops.layer.prefill_positions(seq_info)
        t = sum(new)
        xq = torch.randn(t, HQ, D, generator=g).to(torch.bfloat16)
        xk = torch.randn(t, HKV, D, generator=g).to(torch.bfloat16)
        xv = torch.randn(t, HKV, D, generator=g).to(torch.bfloat16)
        tbl = table[lanes]
        bias = ops.AttnBias.from_seqlens([n for _, n in seq_info], [a + b for a, b in seq_info],
                                         tbl.to(DEV), PAGE)
        out = ops.gqa_attention(
            xq.to(DEV), xk.to(DEV), xv.to(DEV), cache, 0, bias, q_pos.to(DEV),
            None if decode else q_batch.to(DEV), None, freqs.to(DEV), window_left,
        )
        want = ref_gqa_attention_layer(
            xq.clone(), xk.clone(), xv, ref_cache, q_pos, None if decode else q_batch, None, freqs,
            bias.q_seqinfo.seqstart.cpu(), bias.k_seqinfo.seqlen.cpu(), tbl, PAGE, window_left,
        )
        assert (out.cpu().float() - want).abs().max().item() <= 2e-2
        for i in lanes:
            lens[i] += new[i]
        _cache_checks(cache.caches[0], ref_cache)
        # keep the two caches in lock step (K rows may differ in the last bit)
        ref_cache.copy_(cache.caches[0].cpu())


def test_decode_layer_replayed_from_a_cuda_graph(ops):
    """Lengths, block table and the live batch size are device tensors that change
    between replays; the captured launches must follow them (generate.py:338-373,
    forward.py:117-131)."""
    g = torch.Generator().manual_seed(123)
    bs, n_pages, cols = 6, 24, 4
    table = torch.randperm(n_pages, generator=g).reshape(bs, cols).to(torch.int32)
    freqs = ref_rope_freqs(D, 1e6)
    cache = ops.RawCache.build_dims(1, HKV, D, n_pages * PAGE, DEV, torch.bfloat16)
    cache.caches[0].copy_(torch.randn(n_pages * PAGE, 2 * HKV * D, generator=g).to(torch.bfloat16))
    ref_cache = cache.caches[0].cpu().clone()

    # graph-stable inputs, like ModelState: lane capacity as the static key bound
    bias = ops.AttnBias.from_seqlens([1] * bs, [cols * PAGE] * bs, table.to(DEV), PAGE)
    seqlen = bias.k_seqinfo.seqlen
    actual = torch.tensor(bs, dtype=torch.int64, device=DEV)
    xq = torch.zeros(bs, HQ, D, device=DEV, dtype=torch.bfloat16)
    xk = torch.zeros(bs, HKV, D, device=DEV, dtype=torch.bfloat16)
    xv = torch.zeros(bs, HKV, D, device=DEV, dtype=torch.bfloat16)
    freqs_d = freqs.to(DEV)

    def step():
        q_seqpos = seqlen - 1  # forward.py:525
        return ops.gqa_attention(xq, xk, xv, cache, 0, bias, q_seqpos, None, actual, freqs_d, 511)

    seqlen.copy_(torch.tensor([5, 5, 5, 5, 5, 5], dtype=torch.int32))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # warm-up outside the capture, as the reference does
    torch.cuda.current_stream().wait_stream(side)
    cache.caches[0].copy_(ref_cache)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()

    for lens, nactive in (([700, 3, 1024, 256, 1, 90], 6), ([701, 4, 1000, 0, 0, 0], 3),
                          ([702, 1, 513, 77, 0, 0], 4)):
        hq_in = torch.randn(bs, HQ, D, generator=g).to(torch.bfloat16)
        hk_in = torch.randn(bs, HKV, D, generator=g).to(torch.bfloat16)
        hv_in = torch.randn(bs, HKV, D, generator=g).to(torch.bfloat16)
        xq.copy_(hq_in)
        xk.copy_(hk_in)
        xv.copy_(hv_in)
        seqlen.copy_(torch.tensor(lens, dtype=torch.int32))
        actual.fill_(nactive)
        graph.replay()
        torch.cuda.synchronize()
        lens_t = torch.tensor(lens, dtype=torch.int32)
        want = ref_gqa_attention_layer(
            hq_in.clone(), hk_in.clone(), hv_in, ref_cache, lens_t - 1, None, nactive, freqs,
            torch.arange(bs + 1, dtype=torch.int32), lens_t, table, PAGE, 511,
        )
        got = out.cpu().float()
        assert (got[:nactive] - want[:nactive]).abs().max().item() <= 2e-2
        # padded lanes (no keys) give zero rows and write nothing
        assert got[nactive:].abs().sum().item() == 0
        _cache_checks(cache.caches[0], ref_cache)
        ref_cache.copy_(cache.caches[0].cpu())


def test_registered_torch_ops_match_the_eager_wrappers(ops):
    """The ops are also registered as ``torch.ops.cwm_b200.*`` for traced or compiled
    code; called through the dispatcher they give the same bits as the wrappers."""
    from tests.helpers import make_problem

    g = torch.Generator().manual_seed(5)
    x = torch.randn(9, 6144, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(6144, generator=g).to(torch.bfloat16).to(DEV)
    assert torch.equal(torch.ops.cwm_b200.rmsnorm(x, w, 1e-5), ops.rmsnorm(x, w, 1e-5))
    h1, h2 = x.clone(), x.clone()
    d = torch.randn(9, 6144, generator=g).to(torch.bfloat16).to(DEV)
    assert torch.equal(torch.ops.cwm_b200.add_rmsnorm(h1, d, w, 1e-5), ops.add_rmsnorm(h2, d, w, 1e-5))
    assert torch.equal(h1, h2)
    r1 = torch.randn(7, 6, 128, generator=g).to(torch.bfloat16).to(DEV)
    r2 = r1.clone()
    pos = torch.arange(7, dtype=torch.int32, device=DEV)
    freqs = ref_rope_freqs(128, 1e6).to(DEV)
    torch.ops.cwm_b200.rope(r1, pos, freqs)
    ops.apply_rope(r2, pos, freqs)
    assert torch.equal(r1, r2)
    p = make_problem([1, 150], [500, 150 + 60], hq=12, hkv=2, seed=77).to(DEV)
    k4, v4 = p.kv_views()
    out_op, lse_op = torch.ops.cwm_b200.paged_attn_fwd(
        p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table, 150, 512, 128**-0.5, -1)
    out, lse = ops.mha_fwd(p.q, k4, v4, p.cu_seqlens_q, None, p.seqused_k, None, 150, 512, 0,
                           p.block_table, 128**-0.5, True, -1, -1)
    assert torch.equal(out_op, out) and torch.equal(lse_op, lse)


def test_packed_layer_with_pinned_host_input_and_output(lib):
    """The packed layer step with its inputs read from, and its result written to,
    pinned host memory by the kernels themselves equals the same step on device
    buffers bit for bit (decode and prefill rows)."""
    import cwm_b200
    from cwm_b200.layer import gqa_attention_packed, prefill_positions

    hq, hkv, d, page = 12, 2, 128, 256
    g = torch.Generator().manual_seed(77)
    for seq_info in ([(300, 1), (1000, 1), (0, 1), (4000, 1)], [(100, 200), (0, 131)]):
        q_lens = [n1 for _, n1 in seq_info]
        kv_lens = [n0 + n1 for n0, n1 in seq_info]
        cols = max((n + page - 1) // page for n in kv_lens)
        n_pages = cols * len(seq_info)
        table = torch.randperm(n_pages, generator=g).reshape(len(seq_info), cols).to(torch.int32).to(DEV)
        rows0 = torch.randn(n_pages * page, 2 * hkv * d, generator=g).to(torch.bfloat16)
        t = sum(q_lens)
        qkv = torch.randn(t, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
        q_batch, q_pos = prefill_positions(seq_info, DEV)
        decode = max(q_lens) == 1
        bias = cwm_b200.AttnBias.from_seqlens(q_lens, kv_lens, table, page)
        freqs = cwm_b200.rope_freqs(d, 1e6).to(DEV)
        results = []
        for pinned in (False, True):
            cache = cwm_b200.RawCache([rows0.to(DEV)], [hkv * d, hkv * d], n_pages * page)
            src = qkv.pin_memory() if pinned else qkv.to(DEV)
            out = torch.zeros(t, hq, d, dtype=torch.bfloat16).pin_memory() if pinned else None
            got = gqa_attention_packed(src, hq, hkv, cache, 0, bias, q_pos,
                                       None if decode else q_batch, None, freqs, -1, out=out)
            torch.cuda.synchronize()
            if pinned:
                assert got.data_ptr() == out.data_ptr() and not got.is_cuda
            results.append((got.cpu().clone(), cache.caches[0].cpu().clone()))
        assert torch.equal(results[0][0].view(torch.int16), results[1][0].view(torch.int16))
        assert torch.equal(results[0][1].view(torch.int16), results[1][1].view(torch.int16))
        assert results[0][0].abs().sum() > 0
