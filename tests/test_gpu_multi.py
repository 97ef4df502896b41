"""Two-GPU tests (skipped on a single GPU): the peer-memory all-reduce kernel against
a sum computed from gathered inputs, eagerly and replayed from a CUDA graph, and a
tensor-parallel decode step of the small decoder with that kernel against the same
step with the process group's all-reduce.  Ranks are child processes, one per GPU,
that finish with: drop the peer mappings, barrier, destroy the process group."""

from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, what: str, results) -> None:
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from cwm_b200 import _lib
        from cwm_b200.tp import Collectives, PeerAllReduce

        if what == "allreduce":
            peer = PeerAllReduce(None, dev)
            g = torch.Generator(device=dev).manual_seed(100 + rank)
            worst = 0.0
            for it, shape in enumerate([(128, 6144), (8, 16), (3, 6144), (128, 6144), (64, 1024)] * 6):
                x = torch.randn(shape, generator=g, device=dev).to(torch.bfloat16)
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                want = torch.stack([p.float() for p in parts]).sum(0)
                got = peer.all_reduce(x).clone()
                worst = max(worst, (got.float() - want).abs().max().item() /
                            max(1.0, want.abs().max().item()))
                # every rank holds the same bits
                mine = got.view(torch.int16).to(torch.int32).sum().reshape(1).float()
                lo, hi = mine.clone(), mine.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                assert lo.item() == hi.item(), f"ranks differ at call {it}"
            assert worst <= 2.0**-7, worst  # one bf16 rounding of the fp32 sum
            # replayed from a graph with fresh inputs each time, product written in place
            coll = Collectives(None, peer)
            a = torch.randn(128, 512, generator=g, device=dev).to(torch.bfloat16)
            w = torch.randn(6144, 512, generator=g, device=dev).to(torch.bfloat16) * 0.05
            coll.linear_all_reduce(a, w)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = coll.linear_all_reduce(a, w)
            for _ in range(20):
                a.copy_(torch.randn(128, 512, generator=g, device=dev))
                graph.replay()
                local = torch.nn.functional.linear(a, w)
                parts = [torch.empty_like(local) for _ in range(world)]
                dist.all_gather(parts, local)
                want = torch.stack([p.float() for p in parts]).sum(0)
                assert (out.float() - want).abs().max().item() <= 2.0**-6 * want.abs().max().item()
            assert _lib.device_status(torch.cuda.current_stream().cuda_stream) == 0
            torch.cuda.synchronize()
            dist.barrier()
            coll.close()
        elif what == "decoder":
            from cwm_b200.decoder import DecoderArgs, DecodeState, ShardedDecoder

            args = DecoderArgs(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=128,
                               ffn_dim=512, vocab_size=1024, local_window=64, page_size=256)
            logits = {}
            for peer_ar in (False, True):
                model = ShardedDecoder(args, rank, world, dev, seed=3, std=0.05,
                                       peer_all_reduce=peer_ar)
                cache = model.build_cache(6 * 256)
                for c in cache.caches:
                    c.copy_(torch.randn(c.shape, generator=torch.Generator().manual_seed(7 + rank))
                            .to(torch.bfloat16))
                table = torch.arange(6, dtype=torch.int32, device=dev).reshape(3, 2)
                state = DecodeState(3, table, 256, dev)
                state.copy_inputs(state.blktbl, torch.tensor([5, 900, 33], dtype=torch.int32, device=dev),
                                  torch.tensor([100, 1, 400], dtype=torch.int32, device=dev))
                logits[peer_ar] = model.decode(state, cache).clone()
                torch.cuda.synchronize()
                dist.barrier()
                if model.coll is not None:
                    model.coll.close()
            scale = logits[False].abs().max().item()
            assert (logits[True] - logits[False]).abs().max().item() <= 2e-2 * scale
            assert _lib.device_status(torch.cuda.current_stream().cuda_stream) == 0
        elif what == "allreduce_add_rmsnorm":
            from cwm_b200.kernels import add_rmsnorm

            peer = PeerAllReduce(None, dev)
            g = torch.Generator(device=dev).manual_seed(300 + rank)
            gw = torch.Generator(device=dev).manual_seed(299)  # the same weights on every rank
            for it, (rows, d) in enumerate([(128, 6144), (4, 256), (16, 1024), (128, 6144),
                                            (2, 8192), (256, 512)] * 3):
                x = torch.randn(rows, d, generator=g, device=dev).to(torch.bfloat16)
                h = torch.randn(rows, d, generator=gw, device=dev).to(torch.bfloat16)
                w = torch.randn(d, generator=gw, device=dev).to(torch.bfloat16)
                # the three separate steps
                h_ref = h.clone()
                want = add_rmsnorm(h_ref, peer.all_reduce(x).clone(), w, 1e-5)
                # one kernel: all rows of the normalised result, own rows of h
                h_own = h.clone()
                got = peer.all_reduce_add_rmsnorm(x, h_own, w, 1e-5).clone()
                assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (it, rows, d)
                lo, hi = rank * rows // world, (rank + 1) * rows // world
                assert torch.equal(h_own[lo:hi].view(torch.int16), h_ref[lo:hi].view(torch.int16))
                other = torch.ones(rows, dtype=torch.bool)
                other[lo:hi] = False
                assert torch.equal(h_own[other].view(torch.int16), h[other].view(torch.int16))
            # replayed from a graph behind the product that feeds it
            coll = Collectives(None, peer)
            a = torch.randn(64, 512, generator=g, device=dev).to(torch.bfloat16)
            wt = torch.randn(1024, 512, generator=gw, device=dev).to(torch.bfloat16) * 0.05
            wn = torch.randn(1024, generator=gw, device=dev).to(torch.bfloat16)
            h = torch.zeros(64, 1024, device=dev, dtype=torch.bfloat16)
            coll.linear_all_reduce_add_rmsnorm(a, wt, h, wn, 1e-5, True)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = coll.linear_all_reduce_add_rmsnorm(a, wt, h, wn, 1e-5, True)
            for _ in range(10):
                a.copy_(torch.randn(64, 512, generator=g, device=dev))
                h.copy_(torch.randn(64, 1024, generator=gw, device=dev))
                h_ref = h.clone()
                graph.replay()
                got = out.clone()  # the eager call below reuses the result buffers
                want = coll.linear_all_reduce_add_rmsnorm(a, wt, h_ref, wn, 1e-5, False)
                assert torch.equal(got.view(torch.int16), want.view(torch.int16))
            assert _lib.device_status(torch.cuda.current_stream().cuda_stream) == 0
            torch.cuda.synchronize()
            dist.barrier()
            coll.close()
        elif what == "decoder_fused":
            from cwm_b200.decoder import DecoderArgs, DecodeState, ShardedDecoder

            args = DecoderArgs(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=128,
                               ffn_dim=512, vocab_size=1024, local_window=64, page_size=256)
            logits = {}
            for fuse in (False, True):
                model = ShardedDecoder(args, rank, world, dev, seed=3, std=0.05,
                                       peer_all_reduce=True, fuse_all_reduce=fuse)
                cache = model.build_cache(8 * 256)
                for c in cache.caches:
                    c.copy_(torch.randn(c.shape, generator=torch.Generator().manual_seed(7 + rank))
                            .to(torch.bfloat16))
                table = torch.arange(8, dtype=torch.int32, device=dev).reshape(4, 2)
                state = DecodeState(4, table, 256, dev)
                state.copy_inputs(state.blktbl,
                                  torch.tensor([5, 900, 33, 77], dtype=torch.int32, device=dev),
                                  torch.tensor([100, 1, 400, 257], dtype=torch.int32, device=dev))
                logits[fuse] = model.decode(state, cache).clone()
                torch.cuda.synchronize()
                dist.barrier()
                model.coll.close()
            # the fused kernel rounds where the separate steps round
            assert torch.equal(logits[True], logits[False])
            assert _lib.device_status(torch.cuda.current_stream().cuda_stream) == 0
        results[rank] = "ok"
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("what", ["allreduce", "decoder", "allreduce_add_rmsnorm",
                                  "decoder_fused"])
def test_two_ranks(lib, what):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, what, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert [results.get(r) for r in range(2)] == ["ok", "ok"]
    assert all(p.exitcode == 0 for p in procs)
