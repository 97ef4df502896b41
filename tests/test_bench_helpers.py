"""Arithmetic of the benchmark's workload builders and byte/FLOP counts (CPU)."""

from __future__ import annotations

import importlib.util
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_decode_lengths_are_seeded_and_in_range():
    a = bench.decode_lengths(64, 4096, 32768, 1002)
    assert a == bench.decode_lengths(64, 4096, 32768, 1002)
    assert len(a) == 64 and min(a) >= 4096 and max(a) <= 32768


def test_block_tables_place_every_page_once():
    lens = [1, 256, 257, 1000]
    table, n_pages = bench.make_tables(lens, 3)
    assert n_pages == 1 + 1 + 2 + 4 and table.shape == (4, 4) and table.dtype == torch.int32
    used = [int(table[b, c]) for b, n in enumerate(lens) for c in range((n + 255) // 256)]
    assert sorted(used) == list(range(n_pages))
    assert int(table[0, 1]) == 0  # unused entries stay 0, as in the reference engine


def test_algorithmic_bytes_and_pairs():
    # 4096 B per attended token per layer at 8 KV heads (K and V, bf16)
    assert bench.decode_bytes([1000], -1, 48, 8) - bench.decode_bytes([999], -1, 48, 8) == 4096
    assert bench.decode_bytes([1000], -1, 6, 1) - bench.decode_bytes([999], -1, 6, 1) == 512
    # a window caps the attended keys
    assert bench.attended(20000, 8191) == 8192 and bench.attended(100, 8191) == 100
    assert bench.decode_bytes([20000], 8191, 48, 8) < bench.decode_bytes([8300], -1, 48, 8)
    # unmasked (query, key) pairs of a chunk: positions n0 .. n0 + n1 - 1 see pos + 1 keys
    assert bench.prefill_pairs([(0, 3)], -1) == 1 + 2 + 3
    assert bench.prefill_pairs([(10, 2)], -1) == 11 + 12
    assert bench.prefill_pairs([(10, 2)], 4) == 5 + 5
    assert bench.prefill_pairs([(0, 3), (1, 1)], 1) == 1 + 2 + 2 + 2


def test_clock_sampler_summary_parses_nvidia_smi_rows():
    s = bench.ClockSampler(0)
    s.samples = [["1755", "1965", "870.1", "Not Active", "Not Active", "Not Active", "Active"],
                 ["1605", "1965", "990.0", "Not Active", "Not Active", "Not Active", "Not Active"],
                 ["1700", "1965", "990.0", "Not Active", "Not Active", "Not Active", "Active"]]
    out = s.summary()
    assert out["sm_mhz"] == 1700 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"]
