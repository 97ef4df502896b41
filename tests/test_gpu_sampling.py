"""The fused sampling kernel (``cwm_sample``) against the oracle.

Integer work is held bit for bit: on probability inputs the kernel must return
exactly the token, the surviving-entry count and the renormalised probability of
the exact integer statement in ``oracle/ref_sampling.py`` (which the CPU tests pin
to the reference's own functions), and the golden outputs of the reference's
``sample`` / ``top_p`` wherever fp32 rounding of the running sums does not decide.
On logit inputs the probabilities are computed inside the kernel (fast exp2), so
the comparison is with the reference's fp32 path: same token on all but boundary
rows, log-probability within 1e-4.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle.ref_sampling import exact_sample, exact_top_p, ref_sample_logits

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "golden"))
from make_sampling_golden import CASES, case_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def smp(lib):
    from cwm_b200 import sampling

    return sampling


@pytest.fixture(scope="module")
def sampling_golden():
    return np.load(ROOT / "golden" / "sampling_golden.npz")


def _check_exact(smp, probs, p, u):
    tok, pr, kept = smp.top_p(probs.to(DEV), p.to(DEV), uniforms=u.to(DEV), return_kept=True)
    tok_s, pr_s = smp.sample(probs.to(DEV), uniforms=u.to(DEV))
    torch.cuda.synchronize()
    for r in range(probs.shape[0]):
        want = exact_top_p(probs[r].numpy(), float(p.reshape(-1)[r]), float(u[r]))
        got = (int(tok[r]), float(pr[r]), int(kept[r]))
        assert got[0] == want[0] and got[2] == want[2], (r, got, want)
        assert got[1] == pytest.approx(want[1], rel=1e-6)
        want_s = exact_sample(probs[r].numpy(), float(u[r]))
        assert int(tok_s[r]) == want_s[0], (r, int(tok_s[r]), want_s)
        assert float(pr_s[r]) == pytest.approx(want_s[1], rel=1e-6)
    return tok.cpu(), pr.cpu(), tok_s.cpu(), pr_s.cpu()


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_probability_inputs_match_exact_statement_and_reference(smp, sampling_golden, case):
    name, rows, vocab, seed, scale, temp = case
    _, probs, p, u = case_inputs(rows, vocab, seed, scale, temp)
    tok, pr, tok_s, pr_s = _check_exact(smp, probs, p, u)
    # the reference's own outputs (fp32 running sums): equal except where rounding decides
    ref_tok = torch.from_numpy(sampling_golden[f"{name}_top_p_tokens"])
    same = tok == ref_tok
    assert int(same.sum()) >= rows - 1
    ref_pr = torch.from_numpy(sampling_golden[f"{name}_top_p_probs"])
    assert torch.allclose(pr[same], ref_pr[same], rtol=2e-5, atol=1e-9)
    ref_tok_s = torch.from_numpy(sampling_golden[f"{name}_sample_tokens"])
    assert int((tok_s == ref_tok_s).sum()) >= rows - 1


def test_ties_zeros_and_threshold_edges(smp):
    rows = [
        ([0.25, 0.25, 0.25, 0.25], 0.5),
        ([0.1, 0.6, 0.0, 0.3], 0.0),
        ([0.1, 0.6, 0.0, 0.3], 1.0),
        ([0.1, 0.6, 0.0, 0.3], 0.6),
        ([0.0, 0.0, 1.0, 0.0], 0.9),
        ([0.5, 0.5, 0.0, 0.0], 0.4),
    ]
    for u in (0.0, 0.2, 0.34, 0.5, 0.67, 0.999):
        probs = torch.tensor([r for r, _ in rows], dtype=torch.float32)
        p = torch.tensor([[q] for _, q in rows], dtype=torch.float32)
        _check_exact(smp, probs, p, torch.full((len(rows),), u))
    # many equal entries (a uniform row) and an unaligned, ragged vocabulary
    probs = torch.full((3, 5001), 1.0 / 5001)
    _check_exact(smp, probs, torch.tensor([[0.3], [0.9], [1.0]]), torch.tensor([0.1, 0.77, 0.9999]))


def test_unaligned_rows_take_the_scalar_path(smp):
    g = torch.Generator().manual_seed(3)
    big = torch.softmax(torch.randn(5, 1537 + 3, generator=g) * 3, dim=-1)
    view = big[:, 1:1538]  # rows start 4 bytes off a 16-byte boundary, stride 1540
    view = view / view.sum(-1, keepdim=True)
    dev_big = torch.zeros(5, 1540, device=DEV)
    dev_view = dev_big[:, 1:1538]
    dev_view.copy_(view)
    u = torch.rand(5, generator=g)
    p = torch.tensor([0.2, 0.5, 0.9, 0.99, 1.0])
    tok, pr, kept = smp.top_p(dev_view, p.to(DEV), uniforms=u.to(DEV), return_kept=True)
    for r in range(5):
        want = exact_top_p(view[r].contiguous().numpy(), float(p[r]), float(u[r]))
        assert (int(tok[r]), int(kept[r])) == (want[0], want[2])


def test_full_vocabulary_batch_is_exact_and_repeatable(smp):
    g = torch.Generator().manual_seed(8)
    rows, vocab = 128, 128256
    logits = torch.randn(rows, vocab, generator=g) * 2.5
    probs = torch.softmax(logits / 0.7, dim=-1)
    u = torch.rand(rows, generator=g)
    p = torch.tensor([[0.9], [0.95], [0.5], [1.0]]).repeat(rows // 4, 1)
    d_probs, d_p, d_u = probs.to(DEV), p.to(DEV), u.to(DEV)
    tok, pr, kept = smp.top_p(d_probs, d_p, uniforms=d_u, return_kept=True)
    tok2, pr2, kept2 = smp.top_p(d_probs, d_p, uniforms=d_u, return_kept=True)
    assert torch.equal(tok, tok2) and torch.equal(pr, pr2) and torch.equal(kept, kept2)
    for r in (0, 1, 2, 3, 64, 127):
        want = exact_top_p(probs[r].numpy(), float(p[r]), float(u[r]))
        assert (int(tok[r]), int(kept[r])) == (want[0], want[2])
        assert float(pr[r]) == pytest.approx(want[1], rel=1e-6)


def test_logit_inputs_follow_the_reference_path(smp):
    g = torch.Generator().manual_seed(9)
    rows, vocab = 64, 32000
    logits = torch.randn(rows, vocab, generator=g) * 3
    temps = torch.tensor([0.7, 1.0, 1.3, 0.2]).repeat(rows // 4)
    top_ps = torch.tensor([0.9, 1.0, 0.5, 0.95]).repeat(rows // 4)
    u = torch.rand(rows, generator=g)
    for tp in (top_ps, None):
        want_tok, want_lp = ref_sample_logits(logits, temps, tp, True, u)
        tok, lp = smp.sample_logits(logits.to(DEV), temps.to(DEV), None if tp is None else tp.to(DEV),
                                    True, uniforms=u.to(DEV))
        same = tok.cpu() == want_tok
        assert int(same.sum()) >= rows - 2, int(same.sum())
        assert (lp.cpu()[same] - want_lp[same]).abs().max().item() <= 1e-4
    tok, lp = smp.sample_logits(logits.to(DEV), temps.to(DEV), None, False)
    assert torch.equal(tok.cpu(), logits.argmax(-1)) and lp.abs().sum().item() == 0
    # probabilities computed inside the kernel agree with torch's softmax fed to the same kernel
    probs = torch.softmax(logits.to(DEV) / temps.to(DEV)[:, None], dim=-1)
    tok_p, _ = smp.top_p(probs, top_ps.to(DEV), uniforms=u.to(DEV))
    tok_l, _ = smp.sample_logits(logits.to(DEV), temps.to(DEV), top_ps.to(DEV), True,
                                 uniforms=u.to(DEV))
    assert int((tok_p == tok_l).sum()) >= rows - 2


def test_argument_errors(smp):
    x = torch.rand(2, 10, device=DEV)
    with pytest.raises(ValueError):
        smp.sample(x.double())
    with pytest.raises(ValueError):
        smp.sample(x, uniforms=torch.rand(3, device=DEV))
    with pytest.raises(ValueError):
        smp.top_p(torch.rand(1, 200000, device=DEV), 0.9)
    with pytest.raises(RuntimeError):
        smp.sample(torch.rand(2, 10))
