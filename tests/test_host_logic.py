"""Host-side mirror of the reference interface: metadata, cache layout, layer
rules and argument validation (all on the CPU; nothing is launched)."""

from __future__ import annotations

import pytest
import torch

import cwm_b200
from cwm_b200.layer import prefill_positions
from cwm_b200.tp import shard_cache_rows, shard_heads
from oracle import ref_rope_freqs


def test_attn_bias_fields_used_by_the_forward_pass():
    tbl = torch.zeros(3, 5, dtype=torch.int32)
    bias = cwm_b200.AttnBias.from_seqlens([4, 1, 7], [10, 1, 7], tbl, 256)
    assert bias.q_seqinfo.seqstart.tolist() == [0, 4, 5, 12]
    assert bias.q_seqinfo.seqstart.dtype == torch.int32
    assert bias.q_seqinfo.seqstart_py == [0, 4, 5, 12] and bias.q_seqinfo.max_seqlen == 7
    assert bias.k_seqinfo.seqlen.tolist() == [10, 1, 7] and bias.k_seqinfo.seqlen_py == [10, 1, 7]
    assert bias.k_seqinfo.max_seqlen == 10 and bias.page_size == 256
    assert bias.block_tables is tbl
    # the decode loop mutates the length tensor in place between graph replays
    ref = bias.k_seqinfo.seqlen
    bias.k_seqinfo.seqlen.copy_(torch.tensor([11, 2, 8], dtype=torch.int32))
    assert ref.tolist() == [11, 2, 8]
    bias.q_seqinfo.to("cpu")
    bias.k_seqinfo.to("cpu")
    with pytest.raises(ValueError):
        cwm_b200.AttnBias.from_seqlens([1], [1, 2], tbl, 256)
    with pytest.raises(ValueError):
        cwm_b200.AttnBias.from_seqlens([1, 1, 1], [1, 1, 1], tbl.long(), 256)


def test_decode_state_metadata_like_model_state():
    """ModelState builds its mask with the lane capacity as key length
    (forward.py:69-75): max_seqlen_k is a static bound, not the true maximum."""
    tbl = torch.zeros(4, 8, dtype=torch.int32)
    bias = cwm_b200.AttnBias.from_seqlens([1] * 4, [8 * 256] * 4, tbl, 256)
    assert bias.k_seqinfo.max_seqlen == 2048 and bias.q_seqinfo.max_seqlen == 1
    assert bias.q_seqinfo.seqstart.tolist() == [0, 1, 2, 3, 4]


def test_raw_cache_layout_and_views():
    cache = cwm_b200.RawCache.build_dims(3, 2, 128, 1024, "cpu", torch.bfloat16)
    assert len(cache.caches) == 3 and cache.caches[0].shape == (1024, 2 * (128 + 128))
    k, v = cache.cache_kv(1)
    assert k.shape == (1024, 256) and v.shape == (1024, 256)
    assert k.stride() == (512, 1) and v.data_ptr() == k.data_ptr() + 256 * 2
    k4 = k.reshape(-1, 256, 2, 128)
    assert k4.stride() == (256 * 512, 512, 128, 1) and k4.data_ptr() == k.data_ptr()
    assert cache.bytes_per_token() == 3 * 512 * 2
    win = cache.view(256, 512)
    wk, _ = win.cache_kv(0)
    assert wk.shape[0] == 512 and wk.data_ptr() == cache.caches[0].data_ptr() + 256 * 512 * 2
    with pytest.raises(ValueError):
        cache.view(600, 600)
    cache.caches[2].fill_(1)
    cache.clear()
    assert cache.caches[2].abs().sum() == 0
    like = cwm_b200.RawCache.build_like(cache, 64, device="cpu")
    assert like.caches[1].shape == (64, 512) and like.split == cache.split

    class _Attn:
        n_kv_heads = 2

    class _Layer:
        attention = _Attn()

    class _Model:
        kv_lora_rank, qk_head_dim, head_dim, n_layers = 0, 128, 128, 2
        layers = [_Layer(), _Layer()]

    built = cwm_b200.RawCache.build(_Model(), 16, "cpu", torch.float16)
    assert built.caches[0].shape == (16, 512) and built.caches[0].dtype == torch.float16
    _Model.kv_lora_rank = 512
    with pytest.raises(NotImplementedError):
        cwm_b200.RawCache.build(_Model(), 16)


def test_window_rule_and_rope_freqs():
    # 3 local : 1 global, last layer global (transformer.py:79-85)
    lefts = [cwm_b200.window_size_left(i, 64, 4, 8192) for i in range(64)]
    assert lefts[0] == -1 and lefts[1] == lefts[2] == lefts[3] == 8191 and lefts[4] == -1
    assert lefts[63] == -1 and lefts[62] == 8191
    assert sum(1 for v in lefts if v < 0) == 17
    assert cwm_b200.window_size_left(63, 64, 4, 8192, global_last_layer=False) == 8191
    assert cwm_b200.window_size_left(0, 64, 4, 8192, global_window=131072) == 131071
    assert cwm_b200.window_size_left(5, 64, 1, None) == -1
    f = cwm_b200.rope_freqs(128, 1e6)
    assert torch.equal(f, ref_rope_freqs(128, 1e6)) and f.dtype == torch.float32
    sc = dict(low_freq_factor=1, high_freq_factor=4, old_context_len=8192, scale_factor=8)
    assert torch.equal(cwm_b200.rope_freqs(128, 5e5, sc), ref_rope_freqs(128, 5e5, sc))


def test_prefill_positions():
    q_batch, q_pos = prefill_positions([(0, 3), (5, 2), (7, 0), (1, 1)])
    assert q_batch.tolist() == [0, 0, 0, 1, 1, 3] and q_pos.tolist() == [0, 1, 2, 5, 6, 1]
    assert q_batch.dtype == torch.int32 and q_pos.dtype == torch.int32


def test_validation_raises_before_any_launch():
    """Argument errors are ValueError, as in the reference wrappers; they are found
    on the host, so CPU tensors are enough to trigger them."""
    x = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    pos = torch.zeros(4, dtype=torch.int32)
    freqs = torch.zeros(64)
    with pytest.raises(ValueError):
        cwm_b200.apply_rope(x[:, :, :64], pos, freqs)
    with pytest.raises(ValueError):
        cwm_b200.apply_rope(x, pos.long(), freqs)
    with pytest.raises(ValueError):
        cwm_b200.rmsnorm(torch.zeros(4, 8), torch.zeros(4), 1e-5)
    with pytest.raises(ValueError):
        cwm_b200.rmsnorm(torch.zeros(4, 8), torch.zeros(8, dtype=torch.float16), 1e-5)
    src, dst = torch.zeros(4, 64), torch.zeros(32, 64)
    tbl = torch.zeros(4, 2, dtype=torch.int32)
    with pytest.raises(ValueError):
        cwm_b200.paged_memcpy(src, dst, tbl, pos, (2, 2), None, None, 16)
    with pytest.raises(ValueError):
        cwm_b200.paged_memcpy(src, dst, tbl, pos, None, pos, torch.tensor(2), 16)
    with pytest.raises(ValueError):
        cwm_b200.paged_memcpy(src, dst, tbl, pos, None, None, torch.tensor(2.0), 16)
    # valid arguments on CPU tensors: there is no CPU implementation to fall back to
    with pytest.raises(RuntimeError):
        cwm_b200.paged_memcpy(src, dst, tbl, pos, None, None, None, 16)
    with pytest.raises(RuntimeError):
        cwm_b200.rmsnorm(torch.zeros(4, 8), torch.zeros(8), 1e-5)


def test_head_sharding_arithmetic():
    for world in (1, 2, 4, 8):
        shards = [shard_heads(r, world, 48, 8) for r in range(world)]
        assert [s.n_kv for s in shards] == [8 // world] * world
        assert [s.n_q for s in shards] == [48 // world] * world
        assert shards[0].q_begin == 0 and shards[-1].q_end == 48
        for a, b in zip(shards, shards[1:]):
            assert a.q_end == b.q_begin and a.kv_end == b.kv_begin
        # every query head reads a KV head of its own rank
        for s in shards:
            for h in range(s.q_begin, s.q_end):
                assert s.kv_begin <= h // 6 < s.kv_end
    with pytest.raises(ValueError):
        shard_heads(0, 3, 48, 8)
    with pytest.raises(ValueError):
        shard_heads(2, 2, 48, 8)
    rows = torch.arange(4 * 8 * 2 * 4, dtype=torch.float32).reshape(4, 8 * 2 * 4)
    local = shard_cache_rows(rows, shard_heads(1, 4, 48, 8), 8, 4)
    assert local.shape == (4, 2 * 2 * 4)
    assert torch.equal(local[:, :8], rows[:, 8:16]) and torch.equal(local[:, 8:], rows[:, 40:48])


def test_prefill_chunks_match_the_reference_loop():
    """Chunk splitting for prompts longer than the prefill budget, against a literal
    restatement of the reference's loop, plus its invariants."""
    import random

    from oracle import ref_prefill_splits

    rng = random.Random(3)
    for _ in range(300):
        lanes = rng.randint(1, 6)
        seq_info = [(rng.randint(0, 50), rng.randint(1, 40)) for _ in range(lanes)]
        budget = rng.randint(2, 30)
        calls = cwm_b200.prefill_chunks(seq_info, budget)
        assert calls == ref_prefill_splits(seq_info, budget)
        total = sum(n for _, n in seq_info)
        # the calls tile the concatenated tokens, none exceeds the budget
        assert calls[0][0] == 0 and calls[-1][1] == total
        for (f0, l0, _, info0), (f1, _, _, _) in zip(calls, calls[1:]):
            assert l0 == f1
        for f, l, _, info in calls:
            assert 0 < l - f <= budget and sum(n for _, n in info) == l - f
            # a one-token lane whose end coincides with a cut is passed with zero new
            # tokens and fed in the next call (the reference does the same)
            assert all(n >= 0 for _, n in info)
        # every lane ends with all its tokens cached-or-fed, positions contiguous
        fed = {}
        for _, _, lane0, info in calls:
            for k, (cached, n) in enumerate(info):
                lane = lane0 + k
                assert cached == seq_info[lane][0] + fed.get(lane, 0)
                fed[lane] = fed.get(lane, 0) + n
        assert all(fed[i] == n for i, (_, n) in enumerate(seq_info))
    with pytest.raises(ValueError):
        cwm_b200.prefill_chunks([(0, 5)], 1)
    with pytest.raises(ValueError):
        cwm_b200.prefill_chunks([(0, 0)], 8)
