"""GPU parity of the helper kernels (rope, rmsnorm, paged_memcpy, fused rotate +
cache write) through the C ABI: against the golden vectors of the reference's
Triton kernels and against the CPU oracle on seeded inputs."""

from __future__ import annotations

import pytest
import torch

from oracle import ref_paged_memcpy, ref_rmsnorm, ref_rope, ref_rope_freqs
from tests.test_oracle_golden import MEMCPY_CASES, _memcpy_case

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops(lib):
    import cwm_b200

    return cwm_b200


def _status(lib_mod=None):
    from cwm_b200 import _lib

    return _lib.device_status(torch.cuda.current_stream().cuda_stream)


# ------------------------------------------------------------------------ rope
def test_rope_golden_fp32(ops, golden):
    for name in ("small", "grouped"):
        x = torch.from_numpy(golden[f"rope_{name}_x"].copy()).to(DEV)
        pos = torch.from_numpy(golden[f"rope_{name}_pos"]).to(DEV)
        freqs = torch.from_numpy(golden[f"rope_{name}_freqs"]).to(DEV)
        want = torch.from_numpy(golden[f"rope_{name}_out"])
        ops.apply_rope(x, pos, freqs)
        err = (x.cpu() - want).abs().max().item()
        assert err <= 2e-6, (name, err)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,h", [(1, 48), (64, 8), (300, 48), (2048, 6), (5, 1)])
def test_rope_vs_oracle(ops, dtype, n, h):
    g = torch.Generator().manual_seed(n * 100 + h)
    x = torch.randn(n, h, 128, generator=g).to(dtype)
    pos = torch.randint(-1, 131072, (n,), generator=g, dtype=torch.int32)
    freqs = ref_rope_freqs(128, 1e6)
    xg = x.to(DEV)
    ops.apply_rope(xg, pos.to(DEV), freqs.to(DEV))
    exact = ref_rope(x, pos, freqs)  # x now holds the oracle's rounded result
    got = xg.cpu()
    # tolerance of the path: max-abs 2e-2 against the fp32 oracle
    assert (got.float() - exact).abs().max().item() <= 2e-2
    # and in practice no more than one rounding step away from the rounded oracle
    ulp = torch.finfo(dtype).eps * exact.abs().clamp_min(1e-3)
    assert ((got.float() - x.float()).abs() <= ulp).all()


def test_rope_rejects_bad_arguments(ops):
    x = torch.zeros(4, 2, 128, device=DEV, dtype=torch.bfloat16)
    pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    freqs = torch.zeros(64, device=DEV)
    with pytest.raises(ValueError):
        ops.apply_rope(x[:, :, ::2], pos, freqs[:32])
    with pytest.raises(ValueError):
        ops.apply_rope(x, pos[:3], freqs)
    with pytest.raises(ValueError):
        ops.apply_rope(x, pos, freqs[:10])
    with pytest.raises(ValueError):
        ops.apply_rope(x.reshape(8, 128), pos, freqs)


# --------------------------------------------------------------------- rmsnorm
def test_rmsnorm_golden_fp32(ops, golden):
    for name in ("cwm", "odd"):
        x = torch.from_numpy(golden[f"rms_{name}_x"]).to(DEV)
        w = torch.from_numpy(golden[f"rms_{name}_w"]).to(DEV)
        want = torch.from_numpy(golden[f"rms_{name}_out"])
        got = ops.rmsnorm(x, w, float(golden[f"rms_{name}_eps"])).cpu()
        assert torch.allclose(got, want, rtol=2e-5, atol=2e-6), (name, (got - want).abs().max())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n,d", [(1, 6144), (257, 6144), (33, 128), (7, 100), (3, 16384), (2, 24584)])
def test_rmsnorm_vs_oracle(ops, dtype, n, d):
    g = torch.Generator().manual_seed(n + d)
    x = (torch.randn(n, d, generator=g) * 2).to(dtype)
    w = torch.randn(d, generator=g).to(dtype)
    got = ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-5).cpu()
    want = ref_rmsnorm(x, w, 1e-5)
    assert got.dtype == dtype and got.shape == x.shape
    err = (got.float() - want).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.abs().max().item() / 4), err
    # relative: within one rounding step of the output dtype
    rel = ((got.float() - want).abs() / want.abs().clamp_min(1e-2)).max().item()
    assert rel <= 2 * torch.finfo(dtype).eps + 1e-5, rel


def test_rmsnorm_rejects_bad_arguments(ops):
    x = torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.rmsnorm(x.t(), w, 1e-5)
    with pytest.raises(ValueError):
        ops.rmsnorm(x, w[:32], 1e-5)
    with pytest.raises(ValueError):
        ops.rmsnorm(x[0], w, 1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n,d", [(128, 6144), (1, 6144), (33, 128), (5, 8192)])
def test_add_rmsnorm_equals_add_then_rmsnorm(ops, dtype, n, d):
    """The fused residual add + normalisation leaves exactly what ``h.add_(delta)``
    followed by ``rmsnorm(h, w, eps)`` leaves, in h and in the output."""
    g = torch.Generator().manual_seed(n * 3 + d)
    h = torch.randn(n, d, generator=g).to(dtype).to(DEV)
    delta = torch.randn(n, d, generator=g).to(dtype).to(DEV)
    w = torch.randn(d, generator=g).to(dtype).to(DEV)
    h_ref = h.clone()
    h_ref.add_(delta)
    want = ops.rmsnorm(h_ref, w, 1e-5)
    got = ops.add_rmsnorm(h, delta, w, 1e-5)
    assert torch.equal(h.view(torch.uint8), h_ref.view(torch.uint8))
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    exact = ref_rmsnorm(h_ref.cpu(), w.cpu(), 1e-5)
    rel = ((got.cpu().float() - exact).abs() / exact.abs().clamp_min(1e-2)).max().item()
    assert rel <= 2 * torch.finfo(dtype).eps + 1e-5


def test_add_rmsnorm_rejects_bad_arguments(ops):
    h = torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.add_rmsnorm(h, h[:2], w, 1e-5)
    with pytest.raises(ValueError):
        ops.add_rmsnorm(h, h.float(), w, 1e-5)
    odd = torch.zeros(4, 100, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError):  # rows that are not multiples of 16 bytes are not built
        ops.add_rmsnorm(odd, odd.clone(), torch.zeros(100, device=DEV, dtype=torch.bfloat16), 1e-5)


# ---------------------------------------------------------------- paged_memcpy
def test_paged_memcpy_golden_bit_exact(ops, golden):
    for name in MEMCPY_CASES:
        c = _memcpy_case(golden, name)
        full = torch.zeros_like(c["full_want"]).to(DEV)
        e = c["src"].shape[1]
        dst = full[:, e:] if c["kv_view"] else full
        bs = None if c["batch_size"] is None else torch.tensor(c["batch_size"], device=DEV)
        sb = None if c["src_batch"] is None else c["src_batch"].to(DEV)
        ops.paged_memcpy(c["src"].to(DEV), dst, c["tbl"].to(DEV), c["pos"].to(DEV), c["shard"],
                         sb, bs, c["page"])
        assert torch.equal(full.cpu().view(torch.uint8), c["full_want"].view(torch.uint8)), name
    assert _status() == 0


@pytest.mark.parametrize("e,dtype", [(1024, torch.bfloat16), (128, torch.bfloat16),
                                     (1030, torch.float16), (33, torch.float32), (7, torch.int8)])
def test_paged_memcpy_vs_oracle(ops, e, dtype):
    g = torch.Generator().manual_seed(e)
    page, n_pages, b, n = 256, 12, 3, 700
    cols = 4
    tbl = torch.randperm(n_pages, generator=g)[: b * cols].reshape(b, cols).to(torch.int32)
    lane = torch.randint(0, b, (n,), generator=g, dtype=torch.int32)
    # unique (lane, pos) pairs
    flat = torch.randperm(b * cols * page, generator=g)[:n]
    lane = (flat // (cols * page)).to(torch.int32)
    pos = (flat % (cols * page)).to(torch.int32)
    if dtype == torch.int8:
        src = torch.randint(-128, 128, (n, e), generator=g, dtype=torch.int8)
    else:
        src = torch.randn(n, e, generator=g).to(dtype)
    full = torch.zeros(n_pages * page, 2 * e + 8, dtype=dtype)
    want = full.clone()
    ref_paged_memcpy(src, want[:, 8 : 8 + e], tbl, pos, None, lane, None, page)
    fg = full.to(DEV)
    ops.paged_memcpy(src.to(DEV), fg[:, 8 : 8 + e], tbl.to(DEV), pos.to(DEV), None, lane.to(DEV),
                     None, page)
    assert torch.equal(fg.cpu().view(torch.uint8), want.view(torch.uint8))


def test_paged_memcpy_batch_size_and_row_sliced_table(ops):
    g = torch.Generator().manual_seed(9)
    page, e = 256, 256
    big_tbl = torch.randperm(40, generator=g).reshape(8, 5).to(torch.int32)
    tbl = big_tbl[2:6]  # a row slice, like the block-table rows handed to prefill
    src = torch.randn(4, e, generator=g).to(torch.bfloat16)
    pos = torch.tensor([0, 255, 256, 1279], dtype=torch.int32)
    for bs_dtype in (torch.int32, torch.int64):
        want = torch.zeros(40 * page, e, dtype=torch.bfloat16)
        ref_paged_memcpy(src, want, tbl, pos, None, None, 3, page)
        dst = torch.zeros_like(want).to(DEV)
        ops.paged_memcpy(src.to(DEV), dst, big_tbl.to(DEV)[2:6], pos.to(DEV), None, None,
                         torch.tensor(3, dtype=bs_dtype, device=DEV), page)
        assert torch.equal(dst.cpu().view(torch.int16), want.view(torch.int16))


def test_paged_memcpy_flags_bad_page_without_writing(ops):
    page, e = 16, 64
    tbl = torch.tensor([[5, 99]], dtype=torch.int32, device=DEV)  # 99 is outside 8 pages
    dst = torch.zeros(8 * page, e, device=DEV, dtype=torch.bfloat16)
    src = torch.ones(2, e, device=DEV, dtype=torch.bfloat16)
    pos = torch.tensor([3, 20], dtype=torch.int32, device=DEV)
    lane = torch.zeros(2, dtype=torch.int32, device=DEV)
    _status()
    ops.paged_memcpy(src, dst, tbl, pos, None, lane, None, page)
    assert _status() & 1
    assert dst[5 * page + 3].eq(1).all() and dst.sum().item() == e


def test_paged_memcpy_rejects_bad_arguments(ops):
    src = torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16)
    dst = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    tbl = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError):
        ops.paged_memcpy(src, dst.float(), tbl, pos, None, None, None, 16)
    with pytest.raises(ValueError):
        ops.paged_memcpy(src, dst[:, :32], tbl, pos, None, None, None, 16)
    with pytest.raises(ValueError):
        ops.paged_memcpy(src, dst, tbl.long(), pos, None, None, None, 16)
    with pytest.raises(ValueError):
        ops.paged_memcpy(src, dst, tbl, pos[:2], None, None, None, 16)
    with pytest.raises(ValueError):
        ops.paged_memcpy(src, dst, tbl, pos, None, None, torch.zeros(1, dtype=torch.int32, device=DEV), 16)
    with pytest.raises(ValueError):
        ops.paged_memcpy(src, dst.t(), tbl, pos, None, None, None, 16)


# ------------------------------------------------------- fused rope + kv write
@pytest.mark.parametrize("hq,hkv", [(48, 8), (6, 1), (12, 2)])
@pytest.mark.parametrize("mode", ["prefill", "decode"])
def test_rope_kv_write_equals_separate_ops(ops, hq, hkv, mode):
    """The fused launch must leave exactly what the four separate calls of
    forward.py:618-632 leave: xq, xk and the cache rows, bit for bit."""
    g = torch.Generator().manual_seed(hq + hkv)
    d, page, n_pages = 128, 256, 24
    if mode == "prefill":
        t, b = 600, 3
        lane = torch.sort(torch.randint(0, b, (t,), generator=g)).values.to(torch.int32)
        pos = torch.cat([torch.arange((lane == i).sum()) + 37 * i for i in range(b)]).to(torch.int32)
        bs = None
    else:
        t, b = 7, 7
        lane = None
        pos = torch.tensor([0, 255, 256, 700, 5, -1, -1], dtype=torch.int32)
        bs = torch.tensor(5, dtype=torch.int64, device=DEV)
    tbl = torch.randperm(n_pages, generator=g)[: b * 3].reshape(b, 3).to(torch.int32)
    xq = torch.randn(t, hq, d, generator=g).to(torch.bfloat16)
    xk = torch.randn(t, hkv, d, generator=g).to(torch.bfloat16)
    xv = torch.randn(t, hkv, d, generator=g).to(torch.bfloat16)
    freqs = ref_rope_freqs(d, 1e6).to(DEV)
    cache_a = torch.zeros(n_pages * page, 2 * hkv * d, device=DEV, dtype=torch.bfloat16)
    cache_b = torch.zeros_like(cache_a)
    lane_g = None if lane is None else lane.to(DEV)

    q1, k1 = xq.to(DEV), xk.to(DEV)
    ops.apply_rope(q1, pos.to(DEV), freqs)
    ops.apply_rope(k1, pos.to(DEV), freqs)
    ck, cv = torch.split(cache_a, [hkv * d, hkv * d], dim=1)
    ops.paged_memcpy(k1.flatten(1, 2), ck, tbl.to(DEV), pos.to(DEV), None, lane_g, bs, page)
    ops.paged_memcpy(xv.to(DEV).flatten(1, 2), cv, tbl.to(DEV), pos.to(DEV), None, lane_g, bs, page)

    q2, k2 = xq.to(DEV), xk.to(DEV)
    ck2, cv2 = torch.split(cache_b, [hkv * d, hkv * d], dim=1)
    ops.rope_kv_write(q2, k2, xv.to(DEV), ck2, cv2, pos.to(DEV), freqs, tbl.to(DEV), lane_g, bs, page)

    assert torch.equal(q1.view(torch.int16), q2.view(torch.int16))
    assert torch.equal(k1.view(torch.int16), k2.view(torch.int16))
    assert torch.equal(cache_a.view(torch.int16), cache_b.view(torch.int16))
    assert cache_b.abs().sum().item() > 0
    assert _status() == 0


@pytest.mark.parametrize("hq,hkv", [(48, 8), (6, 1)])
@pytest.mark.parametrize("mode", ["prefill", "decode"])
def test_packed_qkv_rope_kv_write_equals_the_split_path(ops, hq, hkv, mode):
    """The packed form (one stacked q|k|v projection output, rows read in place, queries
    written to a fresh tensor) must give the queries and cache rows of rope_kv_write on
    the split tensors, bit for bit, and must leave the packed rows untouched."""
    from cwm_b200.attention import qkv_rope_kv_write

    g = torch.Generator().manual_seed(100 + hq)
    d, page, n_pages = 128, 256, 24
    if mode == "prefill":
        t, b = 500, 3
        lane = torch.sort(torch.randint(0, b, (t,), generator=g)).values.to(torch.int32).to(DEV)
        pos = torch.cat([torch.arange((lane == i).sum().item()) + 41 * i for i in range(b)]).to(torch.int32)
        bs = None
    else:
        t, b = 6, 6
        lane = None
        pos = torch.tensor([0, 255, 256, 700, -1, -1], dtype=torch.int32)
        bs = torch.tensor(4, dtype=torch.int64, device=DEV)
    tbl = torch.randperm(n_pages, generator=g)[: b * 3].reshape(b, 3).to(torch.int32).to(DEV)
    width = (hq + 2 * hkv) * d
    # rows wider than the packed heads: the row stride differs from the row length
    buf = torch.randn(t, width + 64, generator=g).to(torch.bfloat16).to(DEV)
    qkv = buf[:, :width]
    before = qkv.clone()
    freqs = ref_rope_freqs(d, 1e6).to(DEV)
    pos_d = pos.to(DEV)
    cache_a = torch.zeros(n_pages * page, 2 * hkv * d, device=DEV, dtype=torch.bfloat16)
    cache_b = torch.zeros_like(cache_a)

    xq, xk, xv = (x.contiguous().view(t, -1, d) for x in
                  torch.split(before, [hq * d, hkv * d, hkv * d], dim=1))
    ck, cv = torch.split(cache_a, [hkv * d, hkv * d], dim=1)
    ops.rope_kv_write(xq, xk, xv, ck, cv, pos_d, freqs, tbl, lane, bs, page)
    ck2, cv2 = torch.split(cache_b, [hkv * d, hkv * d], dim=1)
    q_out = qkv_rope_kv_write(qkv, hq, hkv, ck2, cv2, pos_d, freqs, tbl, lane, bs, page)

    assert q_out.shape == (t, hq, d) and q_out.is_contiguous()
    assert torch.equal(q_out.view(torch.int16), xq.view(torch.int16))
    assert torch.equal(cache_a.view(torch.int16), cache_b.view(torch.int16))
    assert torch.equal(qkv.view(torch.int16), before.view(torch.int16))
    assert cache_b.abs().sum().item() > 0
    assert _status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_silu_mul_equals_the_two_torch_ops(ops, dtype):
    """F.silu(x1, inplace=True).mul_(x3) of forward.py:776-781 rounds after each
    of the two steps; the fused kernel rounds the same way."""
    from cwm_b200.attention import silu_mul

    g = torch.Generator().manual_seed(7)
    for t, ffn in ((128, 2688), (3, 8), (1000, 512)):
        x13 = (torch.randn(t, 2 * ffn, generator=g) * 3).to(dtype).to(DEV)
        x1, x3 = x13.clone().chunk(2, dim=1)
        want = torch.nn.functional.silu(x1.contiguous(), inplace=True).mul_(x3)
        got = silu_mul(x13)
        assert got.shape == (t, ffn)
        diff = (got.float() - want.float()).abs()
        # expf and torch's exp may differ in the last bit before the rounding
        step = want.float().abs() * (2.0**-7 if dtype == torch.bfloat16 else 2.0**-10
                                     if dtype == torch.float16 else 2.0**-21) + 1e-30
        assert bool((diff <= step).all())
        if dtype != torch.float32:
            assert (diff > 0).float().mean().item() < 0.01
    with pytest.raises(ValueError):
        silu_mul(torch.zeros(4, 7, device=DEV, dtype=torch.bfloat16))
