"""The give-up path of the attention kernels' bounded waits.

Every wait on a shared-memory barrier inside the decode and prefill kernels is
bounded; when one runs out the kernel records status bit 2, lets its copies in
flight land, frees its tensor memory and returns, so the CUDA context stays usable.
The path is made to run by construction, never by a fault: through
``cwm_test_hooks`` the loader warp of each CTA withholds the loads of its last K/V
tile (fewer memory accesses than a normal launch, none that a normal launch would
not make) and the wait limit is shortened to a fraction of a millisecond, so the
waits for that tile give up.  The call must return, the status word must carry bit
2, and a normal call right afterwards must be correct again.
"""

from __future__ import annotations

import pytest
import torch

from oracle import ref_paged_gqa_attention
from tests.helpers import make_problem

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SHORT_LIMIT = 300_000  # SM clock cycles: about 0.15 ms


def _run(p, window_left=-1):
    import cwm_b200

    pg = p.to(DEV)
    k4, v4 = pg.kv_views()
    max_q = int((p.cu_seqlens_q[1:] - p.cu_seqlens_q[:-1]).max())
    out, _ = cwm_b200.mha_fwd(pg.q, k4, v4, pg.cu_seqlens_q, None, pg.seqused_k, None, max_q,
                              pg.block_table.shape[1] * p.page_size, 0, pg.block_table,
                              p.d**-0.5, True, window_left, -1)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("kind", ["decode", "prefill", "prefill_one_tile"])
def test_wait_that_runs_out_sets_status_and_context_survives(lib, kind):
    from cwm_b200 import _lib

    if kind == "decode":
        p = make_problem([1, 1], [700, 130], hq=12, hkv=2, seed=21)
    elif kind == "prefill":
        p = make_problem([300], [400], hq=12, hkv=2, seed=22)
    else:
        p = make_problem([90], [90], hq=12, hkv=2, seed=23)
    stream = torch.cuda.current_stream().cuda_stream
    good = _run(p)
    assert _lib.device_status(stream) == 0
    k4, v4 = p.kv_views()
    want, _ = ref_paged_gqa_attention(p.q, k4, v4, p.cu_seqlens_q, p.seqused_k, p.block_table,
                                      p.d**-0.5, -1)
    assert (good.cpu().float() - want).abs().max().item() <= 2e-2

    assert lib.cwm_test_hooks(SHORT_LIMIT, 1) == 0
    try:
        _run(p)  # returns: every wait is bounded
        status = _lib.device_status(stream)
    finally:
        assert lib.cwm_test_hooks(0, 0) == 0
    assert status & 2, f"status word {status}: the wait did not run out"

    # the context is intact and the next call is right, bit for bit as before
    again = _run(p)
    assert _lib.device_status(stream) == 0
    assert torch.equal(again.view(torch.int16), good.view(torch.int16))
