"""Generate ``helpers_golden.npz`` from the reference's own Triton kernels.

Run where the reference checkout is importable (it is not needed to *use* the
fixtures)::

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/cwm

The three helpers of ``cwm/fastgen/kernels`` (``apply_rope``, ``rmsnorm``,
``paged_memcpy``) are executed on CPU tensors by the Triton interpreter and
their inputs and outputs are stored.  Floating-point cases use fp32 I/O only:
the interpreter truncates fp32 -> bf16 on store where the GPU rounds to nearest,
so bf16 outputs of the interpreter are not the reference's GPU results.  The
pure-copy kernel is stored in 16-bit as well (bit patterns as int16).

The attention call itself (xformers FlashAttention-3) cannot be run here, so no
attention fixture exists: attention parity is unpinned.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference checkout")
    ap.add_argument("--out", default=str(Path(__file__).with_name("helpers_golden.npz")))
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from cwm.fastgen.kernels import apply_rope, paged_memcpy, rmsnorm

    g = torch.Generator().manual_seed(20250101)
    out: dict[str, np.ndarray] = {}

    # ---- rope ---------------------------------------------------------------
    def rope_case(name: str, n: int, h: int, d: int, theta: float, pos: torch.Tensor) -> None:
        x = torch.randn(n, h, d, generator=g)
        freqs = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
        out[f"rope_{name}_x"] = x.numpy().copy()
        out[f"rope_{name}_pos"] = pos.numpy().copy()
        out[f"rope_{name}_freqs"] = freqs.numpy().copy()
        apply_rope(x, pos, freqs)
        out[f"rope_{name}_out"] = x.numpy().copy()

    # one head per program (n*h < 2048), CWM head_dim, decode-like positions
    rope_case(
        "small", 9, 6, 128, 1e6,
        torch.tensor([0, 1, 2, 255, 256, 8191, 32767, 131071, -1], dtype=torch.int32),
    )
    # grouped branch of the launcher (n*h >= 2048)
    rope_case(
        "grouped", 128, 16, 32, 1e4,
        torch.randint(0, 40000, (128,), generator=g, dtype=torch.int32),
    )

    # ---- rmsnorm ------------------------------------------------------------
    for name, n, d, eps in (("cwm", 5, 6144, 1e-5), ("odd", 7, 100, 1e-6)):
        x = torch.randn(n, d, generator=g) * 3.0
        w = torch.randn(d, generator=g)
        out[f"rms_{name}_x"] = x.numpy().copy()
        out[f"rms_{name}_w"] = w.numpy().copy()
        out[f"rms_{name}_eps"] = np.float64(eps)
        out[f"rms_{name}_out"] = rmsnorm(x, w, eps).numpy().copy()

    # ---- paged_memcpy -------------------------------------------------------
    def memcpy_case(
        name: str, n: int, e: int, page: int, n_pages: int, b: int, dtype: torch.dtype,
        use_src_batch: bool, batch_size: int | None, shard: tuple[int, int] | None,
        kv_view: bool,
    ) -> None:
        cols = n_pages // b
        tbl = torch.randperm(n_pages, generator=g)[: b * cols].reshape(b, cols).to(torch.int32)
        if use_src_batch:
            src_batch = torch.randint(0, b, (n,), generator=g, dtype=torch.int32)
            rows_for_tbl = src_batch
        else:
            assert n <= b
            src_batch = None
            rows_for_tbl = torch.arange(n, dtype=torch.int32)
        # distinct (lane, pos) pairs so that the scatter has no write conflicts
        span = cols * page * (shard[1] if shard else 1)
        flat = torch.randperm(b * span, generator=g)
        pos = torch.empty(n, dtype=torch.int32)
        used: dict[int, set[int]] = {}
        it = iter(flat.tolist())
        for i in range(n):
            lane = int(rows_for_tbl[i])
            while True:
                p = next(it) % span
                if p not in used.setdefault(lane, set()):
                    used[lane].add(p)
                    pos[i] = p
                    break
        src = torch.randn(n, e, generator=g).to(dtype)
        rows = n_pages * page
        if kv_view:
            full = torch.zeros(rows, 2 * e, dtype=dtype)
            dst = full[:, e:]  # the V half of a [K|V] cache row
        else:
            full = torch.zeros(rows, e, dtype=dtype)
            dst = full
        bs = None if batch_size is None else torch.tensor(batch_size, dtype=torch.int64)
        paged_memcpy(src, dst, tbl, pos, shard, src_batch, bs, page)

        def bits(t: torch.Tensor) -> np.ndarray:
            if t.dtype == torch.float32:
                return t.numpy().copy()
            return t.view(torch.int16).numpy().copy()

        out[f"mc_{name}_src"] = bits(src)
        out[f"mc_{name}_tbl"] = tbl.numpy().copy()
        out[f"mc_{name}_pos"] = pos.numpy().copy()
        if src_batch is not None:
            out[f"mc_{name}_src_batch"] = src_batch.numpy().copy()
        out[f"mc_{name}_meta"] = np.array(
            [page, n_pages, b, -1 if batch_size is None else batch_size,
             shard[0] if shard else 0, shard[1] if shard else 1, int(kv_view),
             0 if dtype == torch.float32 else 1],
            dtype=np.int64,
        )
        out[f"mc_{name}_full"] = bits(full)

    memcpy_case("prefill_bf16", 40, 256, 16, 12, 3, torch.bfloat16, True, None, None, True)
    memcpy_case("decode_bf16", 6, 128, 16, 12, 6, torch.bfloat16, False, 4, None, True)
    memcpy_case("shard_f32", 24, 64, 8, 8, 2, torch.float32, True, None, (1, 2), False)
    memcpy_case("wide_f32", 5, 1100, 4, 10, 5, torch.float32, False, None, None, False)

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
