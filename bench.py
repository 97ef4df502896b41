"""Benchmark of the paged-KV attention hot path on B200.

Default workload (N=1): decode attention at scale — batch 64, 48 query / 8 KV
heads, head_dim 128, bf16 cache, contexts log-uniform in [4096, 32768], page 256
with random physical placement, global (full-context) layer.  One step = one pass
of decode attention over the batch for one layer.  With ``--gpus N`` the KV heads
are sharded over N ranks (8/N KV heads and 48/N query heads per GPU, same
sequences and block table on every rank) and no data-path collective is needed.

Prints ONE JSON line: metric ``decode_attn_hbm_gbs`` = algorithmic KV+q+out bytes
per step over all ranks divided by the device time of a step (max over ranks).

``--impl reference`` times the CPU restatement of the reference path (the oracle;
the reference itself has no CPU path and its attention kernel does not run on
this GPU) on the host cores, on a bounded sample of the same workload.

Other workloads (``--workload``) are for profiling: ``decode_local`` (window
8192), ``prefill`` / ``prefill_local`` (chunked prefill, 8 x 2048-token chunks
with cached prefixes), ``small`` (a short decode case for profiler captures).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

HQ, HKV, D, PAGE = 48, 8, 128, 256
WINDOW_LOCAL = 8191
L2_BYTES = 126 * 1024 * 1024
# DRAM bytes moved per algorithmic byte by the decode kernel, from the ncu capture
# summarised in profiles/decode_kernel_small_ncu_full.txt (538.33 MB read + written
# for 527.77 MB algorithmic).  The over-fetch is tile granularity at the ends of a
# context, so it grows in proportion to the work.
DECODE_TRAFFIC_RATIO = 538.33 / 527.77


# ------------------------------------------------------------------ workloads
def decode_lengths(batch: int, lo: int, hi: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    u = torch.empty(batch).uniform_(math.log(lo), math.log(hi), generator=g)
    return [int(round(math.exp(v))) for v in u.tolist()]


def make_tables(kv_lens: list[int], seed: int) -> tuple[torch.Tensor, int]:
    """Block table with random physical page placement; unused entries are 0."""
    g = torch.Generator().manual_seed(seed)
    pages = [(n + PAGE - 1) // PAGE for n in kv_lens]
    n_pages = sum(pages)
    perm = torch.randperm(n_pages, generator=g)
    table = torch.zeros(len(kv_lens), max(pages), dtype=torch.int32)
    ofs = 0
    for b, npg in enumerate(pages):
        table[b, :npg] = perm[ofs : ofs + npg].to(torch.int32)
        ofs += npg
    return table, n_pages


def attended(ctx: int, window_left: int) -> int:
    return ctx if window_left < 0 else min(ctx, window_left + 1)


def decode_bytes(kv_lens: list[int], window_left: int, hq: int, hkv: int) -> int:
    """Algorithmic bytes of one decode-attention pass: attended K and V rows, the
    query and output rows, and the block-table entries and lengths read."""
    kv = sum(attended(n, window_left) for n in kv_lens) * 2 * hkv * D * 2
    qo = len(kv_lens) * hq * D * 2 * 2
    meta = sum((attended(n, window_left) + PAGE - 1) // PAGE for n in kv_lens) * 4 + 8 * len(kv_lens)
    return kv + qo + meta


def prefill_pairs(seq_info: list[tuple[int, int]], window_left: int) -> int:
    total = 0
    for n0, n1 in seq_info:
        if window_left < 0:
            total += sum(range(n0 + 1, n0 + n1 + 1))
        else:
            w = window_left + 1
            total += sum(min(p + 1, w) for p in range(n0, n0 + n1))
    return total


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons while a region runs."""

    FIELDS = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5,
                ).stdout.strip()
                if out:
                    self.samples.append([v.strip() for v in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self) -> "ClockSampler":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=10)

    def summary(self) -> dict:
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [
            n for i, n in enumerate(names)
            if any(len(s) > 3 + i and s[3 + i].lower().startswith("active") for s in self.samples)
        ]
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": reasons,
            "samples": len(self.samples),
        }


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------- CPU baseline
def cpu_decode_baseline(kv_lens, table, cache_rows_fn, window_left, hq, hkv, budget_s, seed):
    """Times the oracle's attention on whole sequences of the workload until about
    ``budget_s`` seconds of CPU work are spent.  ``cache_rows_fn(pages)`` returns
    the cache rows of the given physical pages as a CPU tensor."""
    from oracle import ref_paged_gqa_attention

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    spent, done_bytes, used = 0.0, 0, 0
    while spent < budget_s:
        for b, n in enumerate(kv_lens):
            npg = (n + PAGE - 1) // PAGE
            pages = table[b, :npg].long()
            rows = cache_rows_fn(pages)  # [npg * PAGE, hkv * 2 * D] bf16, local page order
            k, v = torch.split(rows, [hkv * D, hkv * D], dim=1)
            local_tbl = torch.arange(npg, dtype=torch.int32)[None]
            q = torch.randn(1, hq, D, generator=g).to(torch.bfloat16)
            t0 = time.perf_counter()
            ref_paged_gqa_attention(
                q, k.reshape(-1, PAGE, hkv, D), v.reshape(-1, PAGE, hkv, D),
                torch.tensor([0, 1], dtype=torch.int32), torch.tensor([n], dtype=torch.int32),
                local_tbl, D**-0.5, window_left,
            )
            spent += time.perf_counter() - t0
            done_bytes += decode_bytes([n], window_left, hq, hkv)
            used += 1
            if spent >= budget_s:
                break
    return {
        "value": done_bytes / spent / 1e9,
        "unit": "GB/s",
        "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"{used} sequence passes over the {len(kv_lens)} sequences of the workload "
                  f"(whole contexts, cycling), fp32 PyTorch restatement, {spent:.1f} s of CPU time",
    }


def cpu_prefill_baseline(window_left: int, budget_s: float) -> dict:
    """Times the oracle on slices of one prefill sequence-chunk of the workload (256
    queries of a 2048-token chunk on a 6144-token cached prefix, all 48/8 heads) and
    reports FLOP/s over the unmasked pairs; the whole workload scales by pairs."""
    from oracle import ref_paged_gqa_attention

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(3)
    t, n0 = 256, 6144 + 1792  # the last 256 queries of the chunk
    n = n0 + t
    npg = (n + PAGE - 1) // PAGE
    rows = torch.randn(npg * PAGE, HKV * 2 * D, generator=g).to(torch.bfloat16)
    k, v = torch.split(rows, [HKV * D, HKV * D], dim=1)
    q = torch.randn(t, HQ, D, generator=g).to(torch.bfloat16)
    tbl = torch.arange(npg, dtype=torch.int32)[None]
    spent, reps = 0.0, 0
    while spent < budget_s:
        t0 = time.perf_counter()
        ref_paged_gqa_attention(q, k.reshape(-1, PAGE, HKV, D), v.reshape(-1, PAGE, HKV, D),
                                torch.tensor([0, t], dtype=torch.int32),
                                torch.tensor([n], dtype=torch.int32), tbl, D**-0.5, window_left)
        spent += time.perf_counter() - t0
        reps += 1
    flops = 4 * D * HQ * prefill_pairs([(n0, t)], window_left) * reps
    return {
        "value": flops / spent / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"{reps} passes over 256 queries of one 2048-token chunk on 7936 cached tokens "
                  f"(48q/8kv heads), fp32 PyTorch restatement, {spent:.1f} s of CPU time; the "
                  "workload's time is extrapolated by unmasked pairs",
    }


def cpu_decoder_baseline(margs, batch: int, ctx: int, budget_s: float) -> dict:
    """Times the oracle's decode step for ONE local and ONE global layer of the
    unsharded model on 2 sequences, and extrapolates to all layers and the whole
    batch (per-sequence cost times batch: an upper bound on what batching the
    CPU GEMMs could save is not modelled)."""
    from oracle.ref_decoder import ref_decode_step
    from oracle import ref_rope_freqs

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(4)
    sample = 2
    hq, hkv, d = margs.n_heads, margs.n_kv_heads, margs.head_dim
    npg = (ctx + 1 + PAGE - 1) // PAGE

    def layer(window_left):
        def w(*shape):
            return torch.randn(*shape, generator=g) * 0.02
        return {"wq": w(hq * d, margs.dim), "wk": w(hkv * d, margs.dim), "wv": w(hkv * d, margs.dim),
                "wo": w(margs.dim, hq * d), "w13": w(2 * margs.ffn_dim, margs.dim),
                "w2": w(margs.dim, margs.ffn_dim), "attention_norm": torch.ones(margs.dim),
                "ffn_norm": torch.ones(margs.dim), "window_left": window_left}

    weights = {"layers": [layer(-1), layer(margs.local_window - 1)],
               "tok_embeddings": torch.randn(1024, margs.dim, generator=g) * 0.02,
               "output": torch.zeros(8, margs.dim), "norm": torch.ones(margs.dim)}
    caches = [torch.randn(sample * npg * PAGE, hkv * 2 * d, generator=g) for _ in range(2)]
    tbl = torch.arange(sample * npg, dtype=torch.int32).reshape(sample, npg)
    tokens = torch.randint(0, 1024, (sample,), generator=g, dtype=torch.int32)
    seqlen = torch.full((sample,), ctx + 1, dtype=torch.int32)
    freqs = ref_rope_freqs(d, margs.rope_theta)
    spent, reps = 0.0, 0
    while spent < budget_s:
        t0 = time.perf_counter()
        ref_decode_step(weights, tokens, seqlen, tbl, caches, freqs, hq, hkv, d, PAGE,
                        margs.norm_eps)
        spent += time.perf_counter() - t0
        reps += 1
    per_pair = spent / reps  # one global + one local layer, 2 sequences
    n_global = sum(1 for i in range(margs.n_layers)
                   if (margs.global_last_layer and i == margs.n_layers - 1)
                   or i % margs.window_pattern == 0)
    # a local layer costs at most what the timed pair's average does: scale by layers / 2
    step_s = per_pair / 2 * margs.n_layers * (batch / sample)
    return {
        "value": batch / step_s, "unit": "tokens/s", "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"{reps} passes of one global + one local layer of the unsharded model on "
                  f"{sample} sequences of {ctx} tokens, fp32 PyTorch restatement, {spent:.1f} s of "
                  f"CPU time; extrapolated to {margs.n_layers} layers ({n_global} global) and "
                  f"{batch} sequences",
    }


def shared_config(workload: str, batch: int, window_left: int) -> dict:
    """The ``config`` object of the JSON line: what the workload is, identical in the
    B200 arm and the reference arm (arm-specific facts go beside it, not into it)."""
    return {"workload": workload, "batch": batch, "heads": f"{HQ}q/{HKV}kv", "head_dim": D,
            "page_size": PAGE, "window_left": window_left, "kv_dtype": "bf16",
            "placement": "random physical pages"}


def median_and_runs(times_ms: list[float]) -> tuple[float, list[float]]:
    return statistics.median(times_ms), [round(t, 6) for t in times_ms]


def _finish(dist) -> None:
    """End of a multi-rank run: wait for every rank, then leave without tearing the
    communicator down.  Destroying an NCCL communicator whose collectives were
    captured in a CUDA graph can block for ever, and nothing is left to clean up."""
    sys.stdout.flush()
    if dist is None:
        return
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


# ------------------------------------------------------------------------ main
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode_global",
                    choices=["decode_global", "decode_local", "small", "prefill", "prefill_local",
                             "prefill_small", "rmsnorm", "rope_kv_write", "mixed", "mixed_local",
                             "decoder", "sampling"])
    ap.add_argument("--decoder-batch", type=int, default=128)
    ap.add_argument("--decoder-ctx", type=int, default=16384)
    ap.add_argument("--decoder-layers", type=int, default=64)
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the timed region of K steps is run (the median is reported)")
    ap.add_argument("--only-decode", action="store_true",
                    help="default workload without the prefill / decode_local / decoder blocks")
    ap.add_argument("--all-reduce", default="nccl", choices=["nccl", "peer"],
                    help="decoder workload: the process group's all-reduce, or this package's "
                         "peer-memory kernel for the row-parallel sums")
    ap.add_argument("--unfused-all-reduce", action="store_true",
                    help="decoder workload with --all-reduce peer: all-reduce, residual add and "
                         "RMSNorm as three kernels instead of one")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--as-shard", type=int, default=1,
                    help="on one GPU, run the per-GPU share of an N-way KV-head sharding "
                         "(profiling aid; the line says so)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n_gpus = args.gpus
    if world != n_gpus and world > 1:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}")
    if HKV % n_gpus != 0:
        raise SystemExit("--gpus must divide the 8 KV heads")

    window_left = WINDOW_LOCAL if args.workload.endswith("local") else -1
    if args.workload == "decoder":
        return bench_decoder(args, rank, local_rank, world)
    if args.workload.startswith("prefill"):
        print(json.dumps(run_prefill(args, window_left, steps=args.steps,
                                     with_cpu=not args.no_cpu_baseline)))
        return
    if args.workload in ("rmsnorm", "rope_kv_write"):
        return bench_helpers(args)
    if args.workload == "sampling":
        return bench_sampling(args)
    if args.workload.startswith("mixed"):
        return bench_mixed(args, window_left)

    if args.workload == "small":
        kv_lens = decode_lengths(32, 2048, 8192, 1002)
    else:
        kv_lens = decode_lengths(64, 4096, 32768, 1002)
    table, n_pages = make_tables(kv_lens, 1002)
    batch = len(kv_lens)
    workload_name = {
        "decode_global": "config 2: decode attention, batch 64, ctx log-uniform [4096, 32768], "
                         "global layer",
        "decode_local": "config 2: decode attention, batch 64, ctx log-uniform [4096, 32768], "
                        "local layer (window 8192)",
        "small": "profiling case: decode attention, batch 32, ctx log-uniform [2048, 8192]",
    }[args.workload]

    # ------------------------------------------------------------ reference arm
    if args.impl == "reference":
        if rank != 0:
            return
        g = torch.Generator().manual_seed(1002)
        # timing does not depend on the values: every sequence reads a prefix of one
        # random block of the longest context, generated once
        base = torch.randn((max(kv_lens) + PAGE - 1) // PAGE * PAGE, HKV * 2 * D,
                           generator=g).to(torch.bfloat16)

        def rows_fn(pages):
            return base[: len(pages) * PAGE]

        times, vals = [], []
        per_step = max(2.0, min(args.cpu_seconds, 120.0 / max(1, args.steps + args.warmup)))
        res = None
        for i in range(args.warmup + args.steps):
            res = cpu_decode_baseline(kv_lens, table, rows_fn, window_left, HQ, HKV, per_step, i)
            if i >= args.warmup:
                vals.append(res["value"])
        value = statistics.mean(vals)
        res["value"] = value
        total_bytes = decode_bytes(kv_lens, window_left, HQ, HKV)
        print(json.dumps({
            "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": value, "unit": "GB/s",
            "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_bytes / (value * 1e9) * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": shared_config(workload_name, batch, window_left),
            "arm_note": "CPU restatement of the reference path on the host cores; each step "
                        "times a bounded sample and ms_per_step is scaled to the whole batch",
            "cpu_baseline": res,
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
        }))
        return

    # ---------------------------------------------------------------- B200 arm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    line = run_decode(args, rank, local_rank, n_gpus, dist, args.workload, window_left,
                      with_cpu=True)
    # The other two parts of the headline metric ride on the default line.
    if args.workload == "decode_global" and args.as_shard == 1 and not args.only_decode:
        t_extra = time.time()
        if n_gpus == 1:
            loc = run_decode(args, rank, local_rank, 1, None, "decode_local", WINDOW_LOCAL,
                             with_cpu=False, with_e2e=False)
            line["decode_local"] = {k: loc[k] for k in ("value", "unit", "ms_per_step",
                                                        "ms_per_step_runs", "parity")}
            line["decode_local"]["roofline_frac"] = loc["roofline"]["frac"]
            line["prefill"] = {
                "global": prefill_summary(run_prefill(args, -1, steps=5, with_cpu=False)),
                "local": prefill_summary(run_prefill(args, WINDOW_LOCAL, steps=5, with_cpu=False)),
                "note": "config 3 (8 x 8192 new tokens in 2048-token chunks, cached prefixes "
                        "uniform in [0, 16384]); fused rotary + KV write + attention; 5 timed "
                        "steps per chunk call after 3 warm-up steps",
            }
        if n_gpus == 8:
            def summary(dec):
                return {"tokens_per_s": dec["value"], "ms_per_step": dec["ms_per_step"],
                        "ms_per_step_runs": dec["ms_per_step_runs"],
                        "frac_of_hbm_bound": dec["roofline"]["frac"], "parity": dec["parity"],
                        "setup_s": dec["setup_s"], "config": dec["config"],
                        "all_reduce": dec.get("all_reduce")}

            # peer-memory all-reduce fused with the residual add and the norm; if its
            # check against the oracle fails, the line says so and carries the unfused run
            args.all_reduce = "peer"
            try:
                line["decoder"] = summary(run_decoder(args, rank, local_rank, world, dist,
                                                      steps=20, with_cpu=False))
            except DecoderParityError as exc:
                line["decoder_fused_failed"] = str(exc)
                args.unfused_all_reduce = True
                line["decoder"] = summary(run_decoder(args, rank, local_rank, world, dist,
                                                      steps=20, with_cpu=False))
            if not args.unfused_all_reduce:
                args.unfused_all_reduce = True
                line["decoder_unfused"] = summary(run_decoder(args, rank, local_rank, world, dist,
                                                              steps=20, with_cpu=False))
            args.unfused_all_reduce = False
            args.all_reduce = "nccl"
            line["decoder_nccl"] = summary(run_decoder(args, rank, local_rank, world, dist,
                                                       steps=20, with_cpu=False))
        line["extra_blocks_s"] = round(time.time() - t_extra, 1)
    if rank == 0:
        print(json.dumps(line))
    _finish(dist)


def _oracle_decode_rows(row, table, kv_lens, xq, hq_l, hkv_l, window_left, seqs):
    """Oracle output rows of the given sequences (this rank's heads), from the device
    cache rows ``row`` copied to the host page by page."""
    from oracle import ref_paged_gqa_attention

    want = {}
    for b in seqs:
        n = kv_lens[b]
        npg = (n + PAGE - 1) // PAGE
        rows = torch.cat([row[int(pg) * PAGE : (int(pg) + 1) * PAGE] for pg in table[b, :npg]]).cpu()
        k, v = torch.split(rows, [hkv_l * D, hkv_l * D], dim=1)
        out, _ = ref_paged_gqa_attention(
            xq[b : b + 1].cpu(), k.reshape(-1, PAGE, hkv_l, D), v.reshape(-1, PAGE, hkv_l, D),
            torch.tensor([0, 1], dtype=torch.int32), torch.tensor([n], dtype=torch.int32),
            torch.arange(npg, dtype=torch.int32)[None], D**-0.5, window_left)
        want[b] = out[0]
    return want


def run_decode(args, rank, local_rank, n_gpus, dist, workload, window_left, with_cpu=True,
               with_e2e=True) -> dict:
    """Decode attention over the batch for one layer; returns the JSON line."""
    import cwm_b200
    from cwm_b200 import _lib

    dev = torch.device("cuda", local_rank)
    if workload == "small":
        kv_lens = decode_lengths(32, 2048, 8192, 1002)
    else:
        kv_lens = decode_lengths(64, 4096, 32768, 1002)
    table, n_pages = make_tables(kv_lens, 1002)
    batch = len(kv_lens)
    hkv_l, hq_l = HKV // n_gpus, HQ // n_gpus
    if args.as_shard > 1:
        if n_gpus != 1 or HKV % args.as_shard:
            raise SystemExit("--as-shard needs --gpus 1 and a divisor of the 8 KV heads")
        hkv_l, hq_l = HKV // args.as_shard, HQ // args.as_shard

    gen = torch.Generator(device=dev).manual_seed(1002 + rank)
    cache = cwm_b200.RawCache.build_dims(1, hkv_l, D, n_pages * PAGE, dev, torch.bfloat16)
    row = cache.caches[0]
    chunk = 1 << 16
    for r0 in range(0, row.shape[0], chunk):
        blk = row[r0 : r0 + chunk]
        blk.copy_(torch.randn(blk.shape, generator=gen, device=dev, dtype=torch.float32))
    table_d = table.to(dev)
    # metadata of a decode step *before* the new token is appended
    lens_before = [n - 1 for n in kv_lens]
    bias = cwm_b200.AttnBias.from_seqlens([1] * batch, kv_lens, table_d, PAGE)
    freqs = cwm_b200.rope_freqs(D, 1e6).to(dev)
    q_pos = torch.tensor(lens_before, dtype=torch.int32, device=dev)
    xq = torch.randn(batch, hq_l, D, generator=gen, device=dev).to(torch.bfloat16)
    xk = torch.randn(batch, hkv_l, D, generator=gen, device=dev).to(torch.bfloat16)
    xv = torch.randn(batch, hkv_l, D, generator=gen, device=dev).to(torch.bfloat16)
    cache_k, cache_v = cache.cache_kv(0)
    k4 = cache_k.reshape(-1, PAGE, hkv_l, D)
    v4 = cache_v.reshape(-1, PAGE, hkv_l, D)
    # write the step's own token so that the cache is complete
    cwm_b200.rope_kv_write(xq, xk, xv, cache_k, cache_v, q_pos, freqs, table_d, None, None, PAGE)

    def attn_step():
        return cwm_b200.mha_fwd(
            xq, k4, v4, bias.q_seqinfo.seqstart, None, bias.k_seqinfo.seqlen, None, 1,
            bias.k_seqinfo.max_seqlen, 0, table_d, D**-0.5, True, window_left, -1,
        )

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    # The reference engine replays decode from CUDA graphs (generate.py:338-373), one
    # graph holding the attention calls of all layers of a decode step one after
    # another.  So does the timed region: a graph of `per_graph` steps (a divisor of K,
    # at most 10: ten layers' worth), replayed K / per_graph times.  Inside a graph a
    # launch may become resident while the one before drains (programmatic stream
    # serialization), as it does between the kernels of the reference's decode graph.
    per_graph = max(g for g in range(1, 11) if args.steps % g == 0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        attn_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_out, _ = attn_step()
        graph_last = graph_out
        for _ in range(per_graph - 1):
            graph_last, _ = attn_step()
    for _ in range(max(3, -(-args.warmup // per_graph))):
        graph.replay()
    sync_all()

    # ---- parity of what is about to be timed: this rank's output rows of three
    # sequences (shortest, median, longest context) against the oracle on its heads
    order = sorted(range(batch), key=lambda b: kv_lens[b])
    sampled = [order[0], order[batch // 2], order[-1]]
    want = _oracle_decode_rows(row, table, kv_lens, xq, hq_l, hkv_l, window_left, sampled)
    max_abs = max((o[b].cpu().float() - want[b]).abs().max().item()
                  for b in sampled for o in (graph_out, graph_last))
    if not torch.equal(graph_out.view(torch.int16), graph_last.view(torch.int16)):
        raise SystemExit("the first and the last step of the captured graph differ")
    par = torch.tensor([max_abs], device=dev)
    if dist is not None:
        dist.all_reduce(par, op=dist.ReduceOp.MAX)
    max_abs = float(par.item())
    if not max_abs <= 2e-2:
        raise SystemExit(f"parity check failed before timing: max-abs {max_abs} > 2e-2 on "
                         f"sequences {sampled}")

    runs = []
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.repeats):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync_all()
            t0.record()
            for _ in range(args.steps // per_graph):
                graph.replay()
            t1.record()
            sync_all()
            t = torch.tensor([t0.elapsed_time(t1)], device=dev)
            if dist is not None:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            runs.append(float(t.item()) / args.steps)
        # keep the sampler alive for at least a few samples on very short runs
        if sum(runs) * args.steps < 500:
            t_end = time.time() + 0.6
            while time.time() < t_end:
                graph.replay()
            torch.cuda.synchronize()
    ms_per_step, runs = median_and_runs(runs)
    status = _lib.device_status(torch.cuda.current_stream().cuda_stream)
    if status != 0:
        raise SystemExit(f"device status word is {status} after the timed region")

    bytes_rank = decode_bytes(kv_lens, window_left, hq_l, hkv_l)
    bytes_all = bytes_rank * n_gpus
    value = bytes_all / (ms_per_step * 1e-3) / 1e9
    peaks, peak_kind = measured_peaks()
    achieved = bytes_rank / (ms_per_step * 1e-3) / 1e9

    workload_name = {
        "decode_global": "config 2: decode attention, batch 64, ctx log-uniform [4096, 32768], "
                         "global layer",
        "decode_local": "config 2: decode attention, batch 64, ctx log-uniform [4096, 32768], "
                        "local layer (window 8192)",
        "small": "profiling case: decode attention, batch 32, ctx log-uniform [2048, 8192]",
    }[workload]
    line = {
        "metric": "decode_attn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
        "ms_per_step_runs": runs,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": shared_config(workload_name, batch, window_left),
        "arm_note": {"heads_per_gpu": f"{hq_l}q/{hkv_l}kv", "kv_bytes_per_gpu": bytes_rank,
                     **({"as_shard": f"one GPU running the share of 1 of {args.as_shard} ranks"}
                        if args.as_shard > 1 else {}),
                     "launch": f"CUDA graphs of {per_graph} consecutive steps (as the layers of "
                               f"a decode graph follow one another), {args.steps // per_graph} "
                               f"replays = {args.steps} steps per timed region; the region is "
                               f"run {args.repeats} times, ms_per_step is the median",
                     "l2": "inputs larger than L2" if bytes_rank > 2 * L2_BYTES else
                           "inputs not larger than L2 at this sharding",
                     "parallelism": f"tp{n_gpus}"},
        "parity": {"max_abs": max_abs, "sequences": sampled, "tolerance": 2e-2,
                   "against": "CPU oracle on this rank's heads, max over ranks, checked on the "
                              "captured step before timing"},
        "clocks": clocks.summary(),
        "gpu_launches": args.steps * args.repeats,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": int(bytes_rank * DECODE_TRAFFIC_RATIO),
                     "peak_kind": f"of {peak_kind}",
                     "note": "per GPU; events bracket the decode kernels (split-KV merge "
                             "included, one launch per step); traffic is the ncu DRAM "
                             "read+write of a smaller capture scaled by the algorithmic bytes"},
    }
    del graph, graph_out, graph_last

    # -------------------------------------------------- end to end, host buffers
    if with_e2e:
        n_q, n_kv = batch * hq_l * D, batch * hkv_l * D
        width = (hq_l + 2 * hkv_l) * D
        # the step's inputs as the stacked projection output would be: rows [q | k | v]
        h_qkv = torch.randn(batch, width).to(torch.bfloat16).pin_memory()
        h_out = torch.empty(batch, hq_l, D, dtype=torch.bfloat16).pin_memory()
        d_qkv = torch.empty(batch, width, dtype=torch.bfloat16, device=dev)

        def body_zero_copy():
            # the two kernels read the inputs from, and write the result to, pinned host
            # memory themselves: the transfers are inside the kernels
            cwm_b200.layer.gqa_attention_packed(h_qkv, hq_l, hkv_l, cache, 0, bias, q_pos, None,
                                                None, freqs, window_left, out=h_out)

        def body_copies():
            d_qkv.copy_(h_qkv, non_blocking=True)
            out = cwm_b200.layer.gqa_attention_packed(d_qkv, hq_l, hkv_l, cache, 0, bias, q_pos,
                                                      None, None, freqs, window_left)
            h_out.copy_(out, non_blocking=True)

        def time_e2e(step):
            for _ in range(3):
                step()
            vals = []
            for _ in range(args.repeats):
                sync_all()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.steps):
                    step()
                e1.record()
                sync_all()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                if dist is not None:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                vals.append(float(t.item()) / args.steps)
            return statistics.median(vals)

        def as_graph(body):
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                body()

            def step():
                g.replay()
                torch.cuda.current_stream().synchronize()  # the host waits for the result
            return g, step

        def eager_step():
            body_copies()
            torch.cuda.current_stream().synchronize()

        eager_ms = time_e2e(eager_step)
        g_copy, step_copy = as_graph(body_copies)
        copy_ms = time_e2e(step_copy)
        copy_out = h_out.clone()
        g_zero, step_zero = as_graph(body_zero_copy)
        zero_ms = time_e2e(step_zero)
        # both paths leave the same bytes in the host buffer
        if not torch.equal(copy_out.view(torch.int16), h_out.view(torch.int16)):
            raise SystemExit("end-to-end paths disagree on the result in the host buffer")
        h2d = h_qkv.numel() * 2
        d2h = h_out.numel() * 2
        line["e2e"] = {
            "value": bytes_all / (zero_ms * 1e-3) / 1e9, "unit": "GB/s",
            "ms_per_step": zero_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "note": "per step, through cwm_b200.layer.gqa_attention_packed with the step's "
                    "q|k|v rows in a pinned host buffer and a pinned host buffer for the result: "
                    "the rotary + KV-cache-write kernel reads the inputs across the host link, "
                    "the attention kernel stores its output rows across it (no separate copy "
                    "calls); the two launches are replayed as one captured CUDA graph, as the "
                    "reference engine replays its decode step, and the host waits for the "
                    "result every step; the KV cache is device-resident state as in the "
                    "reference engine",
        }
        line["e2e_copy_graph"] = {
            "value": bytes_all / (copy_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": copy_ms,
            "note": "the same step with explicit copies: one host-to-device copy of the pinned "
                    "input buffer, the two kernels on device buffers, one device-to-host copy of "
                    "the output, all four replayed as one graph",
        }
        line["e2e_eager"] = {
            "value": bytes_all / (eager_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": eager_ms,
            "note": "the explicit-copy step issued eagerly (no graph): 2 copies + 2 launches "
                    "through the Python wrappers per step",
        }
        line["gpu_launches_e2e_per_step"] = 2
        del g_copy, g_zero
    if with_cpu and rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        def rows_fn(pages):
            return torch.cat([row[int(pg) * PAGE : (int(pg) + 1) * PAGE] for pg in pages]).cpu()

        line["cpu_baseline"] = cpu_decode_baseline(
            kv_lens, table, rows_fn, window_left, HQ, HKV, args.cpu_seconds, 7
        )
    del cache, row, cache_k, cache_v, k4, v4
    torch.cuda.empty_cache()
    return line


def prefill_summary(line: dict) -> dict:
    r = line["roofline"]
    peaks, _ = measured_peaks()
    return {"tflops": line["value"], "ms": line["ms_per_step"], "frac_burst": r["frac"],
            "frac_sustained": line["value"] / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]),
            "per_chunk_ms": line["arm_note"]["per_chunk_ms"], "parity": line["parity"]}


def run_prefill(args, window_left: int, steps: int, with_cpu: bool) -> dict:
    """Chunked prefill (config 3 shapes): 8 sequences, one 2048-token chunk each per
    step, cached prefixes uniform in [0, 16384] plus the chunk index.  Returns the
    JSON line."""
    import cwm_b200
    from cwm_b200.layer import prefill_positions
    from oracle import ref_paged_gqa_attention, ref_rope

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(1003)
    n0s = torch.randint(0, 16385, (8,), generator=g).tolist()
    peaks, peak_kind = measured_peaks()
    results = []
    parity = 0.0
    small = args.workload == "prefill_small"  # one short call, for profiler captures
    for chunk in range(1 if small else 4):
        seq_info = [(n0 + 2048 * chunk, 2048) for n0 in n0s]
        if small:
            seq_info = [(3072, 1024)] * 4
        kv_lens = [a + b for a, b in seq_info]
        table, n_pages = make_tables(kv_lens, 1003)
        cache = cwm_b200.RawCache.build_dims(1, HKV, D, n_pages * PAGE, dev, torch.bfloat16)
        cache.caches[0].normal_()
        bias = cwm_b200.AttnBias.from_seqlens([n1 for _, n1 in seq_info], kv_lens, table.to(dev),
                                              PAGE)
        q_batch, q_pos = prefill_positions(seq_info, dev)
        freqs = cwm_b200.rope_freqs(D, 1e6).to(dev)
        t = sum(n1 for _, n1 in seq_info)
        xq0 = torch.randn(t, HQ, D, device=dev).to(torch.bfloat16)
        xk0 = torch.randn(t, HKV, D, device=dev).to(torch.bfloat16)
        xv = torch.randn(t, HKV, D, device=dev).to(torch.bfloat16)
        xq, xk = xq0.clone(), xk0.clone()

        def step():
            return cwm_b200.gqa_attention(xq, xk, xv, cache, 0, bias, q_pos, q_batch, None, freqs,
                                          window_left)

        if chunk in (0, 3) or small:
            # parity of one call on fresh inputs: the last 32 query rows of the longest
            # sequence against the oracle (rotary on those rows + attention over the
            # sequence's cache rows as the call left them, new K/V rows included)
            out = step()
            torch.cuda.synchronize()
            b = max(range(len(seq_info)), key=lambda i: kv_lens[i])
            n0b, n1b = seq_info[b]
            npg = (kv_lens[b] + PAGE - 1) // PAGE
            q_hi = sum(n1 for _, n1 in seq_info[: b + 1])
            rows = torch.cat([cache.caches[0][int(pg) * PAGE : (int(pg) + 1) * PAGE]
                              for pg in table[b, :npg]]).cpu()
            k, v = torch.split(rows, [HKV * D, HKV * D], dim=1)
            q_tail = xq0[q_hi - 32 : q_hi].cpu().clone()
            ref_rope(q_tail, torch.arange(n0b + n1b - 32, n0b + n1b, dtype=torch.int32),
                     freqs.cpu())
            want, _ = ref_paged_gqa_attention(
                q_tail, k.reshape(-1, PAGE, HKV, D), v.reshape(-1, PAGE, HKV, D),
                torch.tensor([0, 32], dtype=torch.int32),
                torch.tensor([kv_lens[b]], dtype=torch.int32),
                torch.arange(npg, dtype=torch.int32)[None], D**-0.5, window_left)
            got = out[q_hi - 32 : q_hi].cpu().float()
            parity = max(parity, (got - want).abs().max().item())
            if not parity <= 2e-2:
                raise SystemExit(f"prefill parity check failed: max-abs {parity}")
            xq.copy_(xq0)
            xk.copy_(xk0)
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        flops = 4 * D * HQ * prefill_pairs(seq_info, window_left)
        results.append((ms, flops))
        del cache
    total_ms = sum(r[0] for r in results)
    total_flops = sum(r[1] for r in results)
    tf = total_flops / (total_ms * 1e-3) / 1e12
    extra = {}
    if not small and with_cpu:
        extra["cpu_baseline"] = cpu_prefill_baseline(window_left, args.cpu_seconds)
    torch.cuda.empty_cache()
    return {
        **extra,
        "metric": "prefill_attn_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": total_ms,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": shared_config("config 3: chunked prefill 8 x 8192 tokens in 2048-token chunks, "
                                "fused rotary + KV write + attention", 8, window_left),
        "arm_note": {"per_chunk_ms": [r[0] for r in results]},
        "parity": {"max_abs": parity, "tolerance": 2e-2,
                   "against": "CPU oracle (rotary + attention) on the last 32 query rows of the "
                              "longest sequence, first and last chunk call"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "traffic": None,
                     "peak_kind": f"of {peak_kind}"},
    }


def bench_decoder(args, rank: int, local_rank: int, world: int) -> None:
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    line = run_decoder(args, rank, local_rank, world, dist, steps=args.steps,
                       with_cpu=not args.no_cpu_baseline)
    if rank == 0:
        print(json.dumps(line))
    _finish(dist)


def _gather_cat(t: torch.Tensor, dim: int, world: int, dist) -> torch.Tensor:
    if dist is None or world == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    return torch.cat(parts, dim=dim)


def decoder_parity(margs, rank: int, world: int, dev, dist, ctx: int, collectives: bool,
                   peer: bool = False, fuse: bool = True) -> dict:
    """One decode step of a two-layer model with the real layer shapes (and a small
    vocabulary), tensor-parallel over the same ranks, against the CPU oracle of the
    unsharded model built from the gathered weights and caches: checks sharding,
    all-reduces and the attention kernels together at the shapes that are timed."""
    import dataclasses

    from cwm_b200.decoder import DecodeState, ShardedDecoder
    from oracle.ref_decoder import ref_decode_step

    small = dataclasses.replace(margs, n_layers=2, vocab_size=8192)
    shard_of = world if collectives else 1
    model = ShardedDecoder(small, rank if collectives else 0, shard_of, dev, seed=7,
                           peer_all_reduce=peer and collectives and world > 1,
                           fuse_all_reduce=fuse)
    # a batch that splits over the ranks, so that the check runs the same all-reduce path
    # (fused with the residual add and the norm when the peer kernel is used) as the
    # timed model
    batch = max(2, shard_of)
    cols = (ctx + 2 + PAGE - 1) // PAGE
    n_pages = batch * cols
    cache = model.build_cache(n_pages * PAGE)
    gen = torch.Generator(device=dev).manual_seed(70 + rank)
    for c in cache.caches:
        c.copy_(torch.randn(c.shape, generator=gen, device=dev) * 0.5)
    g = torch.Generator().manual_seed(71)
    table = torch.randperm(n_pages, generator=g).reshape(batch, cols).to(torch.int32)
    tokens = torch.randint(0, small.vocab_size, (batch,), generator=g, dtype=torch.int32)
    seqlen = torch.tensor([ctx + 1, ctx // 3 + 1] + [ctx // (i + 2) + 1 for i in range(2, batch)],
                          dtype=torch.int32)
    before = [c.clone() for c in cache.caches]
    state = DecodeState(batch, table.to(dev), PAGE, dev)
    state.copy_inputs(state.blktbl, tokens.to(dev), seqlen.to(dev))
    logits = model.decode(state, cache)
    torch.cuda.synchronize()

    # full (unsharded) weights and cache rows on every rank, the oracle on rank 0
    hq_l, hkv_l, d = model.shard.n_q, model.shard.n_kv, small.head_dim
    layers = []
    for layer in model.layers:
        wq, wk, wv = model.split_qkv(layer)
        w1, w3 = layer["w13"].chunk(2, dim=0)
        layers.append({
            "wq": _gather_cat(wq, 0, shard_of, dist), "wk": _gather_cat(wk, 0, shard_of, dist),
            "wv": _gather_cat(wv, 0, shard_of, dist), "wo": _gather_cat(layer["wo"], 1, shard_of, dist),
            "w13": torch.cat([_gather_cat(w1, 0, shard_of, dist), _gather_cat(w3, 0, shard_of, dist)]),
            "w2": _gather_cat(layer["w2"], 1, shard_of, dist),
            "attention_norm": layer["attention_norm"], "ffn_norm": layer["ffn_norm"],
            "window_left": layer["window_left"],
        })
    emb = _gather_cat(model.tok_embeddings, 0, shard_of, dist)
    out_w = _gather_cat(model.output, 0, shard_of, dist)
    full_caches = []
    for c in before:
        k, v = torch.split(c, [hkv_l * d, hkv_l * d], dim=1)
        full_caches.append(torch.cat([_gather_cat(k, 1, shard_of, dist),
                                      _gather_cat(v, 1, shard_of, dist)], dim=1))
    result = {"max_abs": None}
    if rank == 0:
        weights = {
            "layers": [{k: (v.float().cpu() if torch.is_tensor(v) else v) for k, v in l.items()}
                       for l in layers],
            "tok_embeddings": emb.float().cpu(), "output": out_w.float().cpu(),
            "norm": model.norm.float().cpu(),
        }
        want = ref_decode_step(weights, tokens, seqlen, table,
                               [c.float().cpu() for c in full_caches], model.freqs.cpu(),
                               small.n_heads, small.n_kv_heads, d, PAGE, small.norm_eps)
        err = (logits.cpu() - want).abs().max().item()
        scale = want.abs().max().item()
        result = {"max_abs": err, "logit_scale": scale, "tolerance": 3e-2 * scale,
                  "against": "CPU oracle decode step of the unsharded two-layer model (real layer "
                             f"shapes, vocabulary 8192, {batch} contexts from {ctx + 1} down) built "
                             "from the gathered weights and cache rows; logits of rank 0"}
        if not err <= 3e-2 * scale:
            result["failed"] = f"decoder parity check failed: max-abs {err} vs scale {scale}"
    # every rank learns the outcome, so that all of them leave (or go on) together
    flag = torch.tensor([1 if "failed" in result else 0], device=dev)
    if dist is not None and collectives:
        dist.broadcast(flag, src=0)
    if model.coll is not None:
        torch.cuda.synchronize()
        model.coll.close()
    del model, cache, before, full_caches, layers, emb, out_w
    torch.cuda.empty_cache()
    if int(flag.item()):
        raise DecoderParityError(result.get("failed", "decoder parity check failed on rank 0"))
    return result


class DecoderParityError(SystemExit):
    """The tensor-parallel decode step disagreed with the CPU oracle; raised on every
    rank after the peer buffers of the checked model were released."""


def run_decoder(args, rank: int, local_rank: int, world: int, dist, steps: int,
                with_cpu: bool) -> dict:
    """Config 5: whole decode step of a CWM-32B-shaped decoder (random bf16 weights),
    tensor-parallel over ``world`` GPUs, batch 128, contexts of 16384 tokens whose
    K/V are random (the prompts are not prefilled: their pages are filled directly),
    one CUDA-graph replay per step; tokens/s = batch * steps / time.  Sampling is
    not part of the step."""
    from cwm_b200.decoder import DecoderArgs, DecodeState, ShardedDecoder

    t_setup = time.time()
    dev = torch.device("cuda", local_rank)
    margs = DecoderArgs(n_layers=args.decoder_layers)
    batch, ctx = args.decoder_batch, args.decoder_ctx
    shard_of = world
    if args.as_shard > 1:
        if world != 1:
            raise SystemExit("--as-shard needs a single process")
        shard_of = args.as_shard
    parity = decoder_parity(margs, rank, world, dev, dist, min(ctx, 16384),
                            collectives=shard_of == world, peer=args.all_reduce == "peer",
                            fuse=not args.unfused_all_reduce)
    total_steps = max(3, args.warmup) + steps * args.repeats + 4
    cols = (ctx + total_steps + PAGE - 1) // PAGE
    n_pages = batch * cols
    kv_gb = n_pages * PAGE * (HKV // shard_of) * 2 * D * 2 * margs.n_layers / 1e9
    free_gb = torch.cuda.mem_get_info(dev)[0] / 1e9
    if kv_gb + 20 > free_gb:
        raise SystemExit(f"decoder workload needs {kv_gb:.0f} GB of KV cache per GPU, "
                         f"{free_gb:.0f} GB free: use more GPUs or smaller --decoder-* values")
    model = ShardedDecoder(margs, rank if shard_of == world else 0, shard_of, dev, seed=5,
                           collectives=shard_of == world,
                           peer_all_reduce=args.all_reduce == "peer" and shard_of == world and world > 1,
                           fuse_all_reduce=not args.unfused_all_reduce)
    cache = model.build_cache(n_pages * PAGE)
    cache.caches[0].normal_()
    for c in cache.caches[1:]:
        c.copy_(cache.caches[0])
    g = torch.Generator().manual_seed(1005)
    table = torch.randperm(n_pages, generator=g).reshape(batch, cols).to(torch.int32).to(dev)
    state = DecodeState(batch, table, PAGE, dev)
    tokens = torch.randint(0, margs.vocab_size, (batch,), generator=g, dtype=torch.int32).to(dev)
    seqlen = torch.full((batch,), ctx + 1, dtype=torch.int32, device=dev)
    state.copy_inputs(state.blktbl, tokens, seqlen)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model.decode(state, cache)
    torch.cuda.current_stream().wait_stream(side)
    sync_all()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        logits = model.decode(state, cache)

    def step():
        graph.replay()
        state.seqlen.add_(1)  # the next token lands one position further

    for _ in range(max(3, args.warmup)):
        step()
    sync_all()
    # latency of one all-reduce of the step's message, 32 in a row inside a graph
    ar_us = None
    if model.coll is not None:
        coll = model.coll
        msg = torch.zeros(batch, margs.dim, dtype=torch.bfloat16, device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            coll.all_reduce(msg)
        torch.cuda.current_stream().wait_stream(side)
        sync_all()
        ar_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(ar_graph):
            for _ in range(32):
                coll.all_reduce(msg)
        ar_graph.replay()
        sync_all()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(5):
            ar_graph.replay()
        a1.record()
        sync_all()
        t_ar = torch.tensor([a0.elapsed_time(a1)], device=dev)
        dist.all_reduce(t_ar, op=dist.ReduceOp.MAX)
        ar_us = float(t_ar.item()) * 1e3 / (5 * 32)
        del ar_graph
    setup_s = time.time() - t_setup
    runs = []
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync_all()
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            sync_all()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if dist is not None:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            runs.append(float(ms.item()) / steps)
    ms_per_step, runs = median_and_runs(runs)
    finite = bool(torch.isfinite(logits).all().item())
    peaks, peak_kind = measured_peaks()
    lefts = [l["window_left"] for l in model.layers]
    kv_bytes = sum(attended(ctx + 1, wl) for wl in lefts) * batch * 2 * (HKV // shard_of) * D * 2
    w_bytes = sum(t.numel() * 2 for l in model.layers for t in l.values() if torch.is_tensor(t))
    w_bytes += model.output.numel() * 2
    bound_ms = (kv_bytes + w_bytes) / (peaks["hbm_gbs"] * 1e9) * 1e3
    line = {
        "metric": "decode_tokens_per_s", "value": batch / (ms_per_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_per_step, "ms_per_step_runs": runs, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config 5: CWM-32B-shaped decoder decode step, random weights",
                   "batch": batch, "context": ctx, "layers": margs.n_layers,
                   "global_layers": sum(1 for v in lefts if v < 0), "parallelism": f"tp{world}",
                   **({"as_shard": f"one GPU running rank 0 of {shard_of}, no collectives"}
                      if shard_of != world else {}),
                   "launch": "one CUDA-graph replay per step", "logits_finite": finite,
                   "sampling": "excluded",
                   "all_reduce": ("peer-memory kernel (cwm_allreduce)" if args.unfused_all_reduce
                                  or batch % world else
                                  "peer-memory kernel fused with the residual add and the RMSNorm "
                                  "after it (cwm_allreduce_add_rmsnorm)")
                                 if args.all_reduce == "peer" and world > 1
                                 else "process group (NCCL)"},
        "parity": parity, "setup_s": round(setup_s, 1),
        "all_reduce": {"us_per_call": ar_us, "bytes": batch * margs.dim * 2,
                       "calls_per_step": 2 * margs.n_layers + 1,
                       "note": "32 back-to-back calls replayed from a graph, max over ranks"},
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "lower_bound_ms": bound_ms, "frac": bound_ms / ms_per_step,
                     "kv_bytes_per_gpu": kv_bytes, "weight_bytes_per_gpu": w_bytes,
                     "peak_kind": f"of {peak_kind}",
                     "note": "lower bound = (attended KV + weights read once) / HBM peak; "
                             "all-reduce time not included"},
    }
    if rank == 0 and world == 1 and with_cpu:  # single-process runs only
        line["cpu_baseline"] = cpu_decoder_baseline(margs, batch, ctx, args.cpu_seconds)
    del graph, logits
    if model.coll is not None:
        sync_all()
        model.coll.close()  # collective: unmap peers, barrier, free
    del model, cache
    torch.cuda.empty_cache()
    return line


def _time_steps(step, steps: int, warmup: int) -> float:
    """Milliseconds per call of ``step`` (CUDA events around ``steps`` calls)."""
    for _ in range(max(3, warmup)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_helpers(args) -> None:
    """HBM-bound helpers at config-4 / config-3 sizes: RMSNorm over [33008, 6144] and
    the fused rotary + KV-cache write of a 16384-token prefill step."""
    import cwm_b200
    from cwm_b200.layer import prefill_positions

    dev = torch.device("cuda", 0)
    peaks, peak_kind = measured_peaks()
    if args.workload == "rmsnorm":
        n, d = 33008, 6144
        x = torch.randn(n, d, device=dev).to(torch.bfloat16)
        w = torch.randn(d, device=dev).to(torch.bfloat16)
        ms = _time_steps(lambda: cwm_b200.rmsnorm(x, w, 1e-5), args.steps, args.warmup)
        nbytes = 2 * n * d * 2 + d * 2
        name = "config 4: RMSNorm (eps 1e-5) over [33008, 6144] bf16"
    else:
        seq_info = [(4096, 2048)] * 8
        kv_lens = [a + b for a, b in seq_info]
        table, n_pages = make_tables(kv_lens, 1003)
        cache = cwm_b200.RawCache.build_dims(1, HKV, D, n_pages * PAGE, dev, torch.bfloat16)
        q_batch, q_pos = prefill_positions(seq_info, dev)
        t = q_pos.shape[0]
        xq = torch.randn(t, HQ, D, device=dev).to(torch.bfloat16)
        xk = torch.randn(t, HKV, D, device=dev).to(torch.bfloat16)
        xv = torch.randn(t, HKV, D, device=dev).to(torch.bfloat16)
        freqs = cwm_b200.rope_freqs(D, 1e6).to(dev)
        ck, cv = cache.cache_kv(0)
        tbl = table.to(dev)
        ms = _time_steps(
            lambda: cwm_b200.rope_kv_write(xq, xk, xv, ck, cv, q_pos, freqs, tbl, q_batch, None,
                                           PAGE),
            args.steps, args.warmup,
        )
        # read q, k, v; write q, k in place; write k, v pages
        nbytes = t * D * 2 * (2 * HQ + 2 * HKV + HKV + 2 * HKV)
        name = "config 3: fused rotary + KV-cache write, 8 x 2048 new tokens, 48q/8kv heads"
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": f"{args.workload}_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "bytes": nbytes},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                     "peak_kind": f"of {peak_kind}"},
    }))


def bench_sampling(args) -> None:
    """Token sampling at the engine's shapes: 128 rows of 128256 fp32 logits,
    temperature 0.7, top-p 0.95 on every row (descending-order draw) and without
    top-p (index-order draw); one launch per call, timed as CUDA-graph replays over
    four copies of the logits in turn.  The algorithmic bytes are one read of the
    logits; the kernel makes several passes, all but the first served by L2 (the
    65.7 MB of one call fit)."""
    from cwm_b200 import sampling
    from oracle.ref_sampling import ref_sample_logits

    dev = torch.device("cuda", 0)
    rows, vocab = 128, 128256
    g = torch.Generator().manual_seed(1006)
    logits_h = torch.randn(rows, vocab, generator=g) * 2.5
    logits = logits_h.to(dev)
    temps = torch.full((rows,), 0.7, device=dev)
    top_ps = torch.full((rows,), 0.95, device=dev)
    u = torch.rand(rows, generator=g).to(dev)
    peaks, peak_kind = measured_peaks()
    nbytes = rows * vocab * 4
    # four copies of the logits (263 MB, more than L2) taken in turn, so that the first
    # pass of every launch reads HBM; the four launches are replayed as one CUDA graph,
    # as the engine's decode step would hold them
    copies = [logits] + [logits.clone() for _ in range(3)]

    def graphed(call) -> float:
        for x in copies:
            call(x)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for x in copies:
                call(x)
        return _time_steps(graph.replay, args.steps, args.warmup) / len(copies)

    out = {}
    for name, call in (
            ("top_p", lambda x: sampling.sample_logits(x, temps, top_ps, True, uniforms=u)),
            ("index_order", lambda x: sampling.sample_logits(x, temps, None, True, uniforms=u)),
            ("greedy", lambda x: sampling.sample_logits(x, temps, None, False))):
        ms = graphed(call)
        out[name] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    # parity on the timed inputs: the reference's fp32 path on 8 of the rows
    tok, _ = sampling.sample_logits(logits, temps, top_ps, True, uniforms=u)
    want, _ = ref_sample_logits(logits_h[:8], temps[:8].cpu(), top_ps[:8].cpu(), True, u[:8].cpu())
    same = int((tok[:8].cpu() == want).sum())
    if same < 7:
        raise SystemExit(f"sampling parity check failed: {same} of 8 tokens agree")
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < min(args.cpu_seconds, 10.0):
        ref_sample_logits(logits_h[:16], temps[:16].cpu(), top_ps[:16].cpu(), True, u[:16].cpu())
        reps += 1
    cpu_s = (time.perf_counter() - t0) / reps / 16 * rows
    print(json.dumps({
        "metric": "sampling_hbm_gbs", "value": out["top_p"]["gbs"], "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": out["top_p"]["ms"],
        "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "sampling: 128 x 128256 fp32 logits, temperature 0.7, top-p 0.95",
                   "bytes": nbytes, "timing": "CUDA-graph replay, 4 logits copies in turn "
                                              "(263 MB, larger than L2)"},
        "modes": out, "parity": {"tokens_equal_of_8": same},
        "cpu_baseline": {"value": nbytes / cpu_s / 1e9, "unit": "GB/s",
                         "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{reps} passes over 16 rows with the torch restatement of the "
                                   "reference path (softmax, sort, cumsum, mask, draw), scaled to "
                                   "128 rows"},
        "roofline": {"bound": "hbm", "achieved": out["top_p"]["gbs"], "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": out["top_p"]["frac"], "traffic": None,
                     "peak_kind": f"of {peak_kind}"},
    }))


def bench_mixed(args, window_left: int) -> None:
    """Config 4: one varlen call with 16 prefill chunks of 2048 tokens (no cached
    prefix) and 240 single-token decodes (contexts lognormal, median 6000, sigma 1,
    clipped to [256, 65536])."""
    import cwm_b200

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(1004)
    z = torch.randn(240, generator=g)
    dec = [int(min(65536, max(256, round(6000 * math.exp(v))))) for v in z.tolist()]
    q_lens = [2048] * 16 + [1] * 240
    kv_lens = [2048] * 16 + dec
    table, n_pages = make_tables(kv_lens, 1004)
    cache = cwm_b200.RawCache.build_dims(1, HKV, D, n_pages * PAGE, dev, torch.bfloat16)
    cache.caches[0].normal_()
    bias = cwm_b200.AttnBias.from_seqlens(q_lens, kv_lens, table.to(dev), PAGE)
    t = sum(q_lens)
    xq = torch.randn(t, HQ, D, device=dev).to(torch.bfloat16)
    ck, cv = cache.cache_kv(0)
    k4, v4 = ck.reshape(-1, PAGE, HKV, D), cv.reshape(-1, PAGE, HKV, D)

    def step():
        return cwm_b200.mha_fwd(
            xq, k4, v4, bias.q_seqinfo.seqstart, None, bias.k_seqinfo.seqlen, None, 2048,
            bias.k_seqinfo.max_seqlen, 0, bias.block_tables, D**-0.5, True, window_left, -1,
        )

    ms = _time_steps(step, args.steps, args.warmup)
    peaks, peak_kind = measured_peaks()
    dec_bytes = decode_bytes(dec, window_left, HQ, HKV)
    flops = 4 * D * HQ * prefill_pairs([(0, 2048)] * 16, window_left)
    bound_ms = dec_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3 + flops / (peaks["bf16_tflops"] * 1e12) * 1e3
    print(json.dumps({
        "metric": "mixed_step_ms", "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": False,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config 4: 16 prefill chunks of 2048 + 240 decodes in one call",
                   "window_left": window_left, "decode_kv_bytes": dec_bytes,
                   "prefill_flops": flops, "sigma": 1.0},
        "roofline": {"bound": "hbm+tensor", "lower_bound_ms": bound_ms, "frac": bound_ms / ms,
                     "peak_kind": f"of {peak_kind}",
                     "note": "lower bound = decode bytes / HBM peak + prefill FLOPs / bf16 peak "
                             "(the two kernels run back to back on one stream)"},
    }))


if __name__ == "__main__":
    main()
