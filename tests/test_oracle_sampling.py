"""The sampling oracle against the reference's own functions.

``tests/golden/sampling_golden.npz`` holds the outputs of the reference's
``sample`` and ``top_p`` (``cwm/fastgen/utils/sampling.py``) on seeded inputs, with
``torch.multinomial`` replaced by an inverse-CDF lookup on stored uniforms (see
``tests/golden/make_sampling_golden.py``).  The fp32 restatement must reproduce
them exactly; the exact integer statement (what the CUDA kernel is held to) must
agree with the restatement wherever fp32 rounding of the running sums does not
decide, which the tests quantify.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle.ref_sampling import (exact_sample, exact_top_p, ref_sample, ref_sample_logits,
                                 ref_top_p, to_units)

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "golden"))
from make_sampling_golden import CASES, case_inputs  # noqa: E402


@pytest.fixture(scope="module")
def sampling_golden():
    return np.load(ROOT / "golden" / "sampling_golden.npz")


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_restatement_reproduces_the_reference(sampling_golden, case):
    name, rows, vocab, seed, scale, temp = case
    _, probs, p, u = case_inputs(rows, vocab, seed, scale, temp)
    assert np.array_equal(u.numpy(), sampling_golden[f"{name}_u"])
    tok, prob = ref_sample(probs.clone(), u)
    assert np.array_equal(tok.numpy(), sampling_golden[f"{name}_sample_tokens"])
    assert np.array_equal(prob.numpy(), sampling_golden[f"{name}_sample_probs"])
    # the reference sorts without asking for stability; on these inputs (no equal
    # probabilities near a draw) the stable order gives the same tokens
    tok, prob, _ = ref_top_p(probs.clone(), p, u)
    assert np.array_equal(tok.numpy(), sampling_golden[f"{name}_top_p_tokens"])
    assert np.array_equal(prob.numpy(), sampling_golden[f"{name}_top_p_probs"])


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_exact_statement_agrees_with_the_reference(sampling_golden, case):
    name, rows, vocab, seed, scale, temp = case
    _, probs, p, u = case_inputs(rows, vocab, seed, scale, temp)
    _, _, kept_ref = ref_top_p(probs.clone(), p, u)
    same_tok = 0
    for r in range(rows):
        row = probs[r].numpy()
        tok, prob, kept = exact_top_p(row, float(p[r]), float(u[r]))
        # the mask: the two running sums differ by fp32 rounding only, so the two
        # surviving sets (prefixes of the descending order) differ by entries whose
        # total probability is within that rounding.  (With p = 1 the reference's
        # fp32 running sum can pass 1.0 and drop a tail of negligible mass, which
        # the exact statement keeps.)
        lo, hi = sorted((kept, int(kept_ref[r])))
        between = np.sort(row.astype(np.float64))[::-1][lo:hi].sum()
        assert between <= 3e-6, (r, kept, int(kept_ref[r]), between)
        if tok == int(sampling_golden[f"{name}_top_p_tokens"][r]):
            same_tok += 1
            assert prob == pytest.approx(float(sampling_golden[f"{name}_top_p_probs"][r]),
                                         rel=2e-5, abs=1e-9)
        else:
            # a different token only where u falls within rounding of an interval
            # end: both tokens are neighbours in the descending order
            order = np.argsort(-row.astype(np.float64), kind="stable")
            pos = {int(t): i for i, t in enumerate(order[: kept + 2])}
            other = int(sampling_golden[f"{name}_top_p_tokens"][r])
            assert abs(pos[tok] - pos[other]) == 1
        tok, prob = exact_sample(row, float(u[r]))
        ref_tok = int(sampling_golden[f"{name}_sample_tokens"][r])
        assert abs(tok - ref_tok) <= 1
        if tok == ref_tok:
            assert prob == pytest.approx(float(sampling_golden[f"{name}_sample_probs"][r]),
                                         rel=2e-5)
    assert same_tok >= rows - 1


def test_units_are_exact_and_monotone():
    p = np.array([0.0, 1e-45, 2.0**-44, 2.0**-43, 3e-10, 0.25, 0.5, 1.0, -0.5], dtype=np.float32)
    u = to_units(p)
    assert list(u[:4]) == [0, 1, 1, 2] and u[-1] == 0
    assert u[5] == 2**42 and u[6] == 2**43 and u[7] == 2**44
    rng = np.random.default_rng(0)
    x = np.sort(rng.random(10000).astype(np.float32) ** 8)
    assert np.all(np.diff(to_units(x).astype(np.int64)) >= 0)


def test_ties_and_edges_of_the_exact_statement():
    # four equal entries: p = 0.5 keeps those whose exclusive sum is <= 0.5: three
    row = np.full(4, 0.25, dtype=np.float32)
    for u, want in ((0.0, 0), (0.34, 1), (0.67, 2), (0.999, 2)):
        tok, prob, kept = exact_top_p(row, 0.5, u)
        assert (tok, kept) == (want, 3) and prob == pytest.approx(1 / 3)
    # p = 0 keeps the single largest entry; p >= 1 keeps every positive entry
    row = np.array([0.1, 0.6, 0.0, 0.3], dtype=np.float32)
    assert exact_top_p(row, 0.0, 0.99)[::2] == (1, 1)
    assert exact_top_p(row, 1.0, 0.99)[::2] == (0, 3)
    assert exact_top_p(row, 0.6, 0.99)[::2] == (3, 2)   # exclusive sums 0, 0.6, 0.9
    assert exact_sample(row, 0.05)[0] == 0 and exact_sample(row, 0.5)[0] == 1
    assert exact_sample(row, 0.71)[0] == 3  # the zero entry is never drawn


def test_sample_logits_restatement_matches_its_parts():
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(6, 500, generator=g) * 3
    temps = torch.tensor([0.7, 1.0, 1.3, 0.2, 0.7, 2.0])
    top_ps = torch.tensor([0.9, 1.0, 0.5, 0.95, 0.1, 1.0])
    u = torch.rand(6, generator=g)
    tok, lp = ref_sample_logits(logits, temps, top_ps, True, u)
    probs = torch.softmax(logits / temps[:, None], dim=-1)
    tok2, pr2, _ = ref_top_p(probs, top_ps[:, None], u)
    assert torch.equal(tok, tok2) and torch.allclose(lp, torch.log(pr2))
    tok, lp = ref_sample_logits(logits, temps, None, False, u)
    assert torch.equal(tok, logits.argmax(-1)) and lp.abs().sum() == 0
