"""Generate ``sampling_golden.npz`` from the reference's own sampling functions.

Run where the reference checkout is readable (it is not needed to *use* the
fixtures)::

    python tests/golden/make_sampling_golden.py --reference /path/to/cwm

``cwm/fastgen/utils/sampling.py`` is loaded from its file (it imports only torch)
and its ``sample`` and ``top_p`` are run on seeded CPU inputs.  The one thing
replaced is the random draw: inside that module ``torch.multinomial`` is swapped
for an inverse-CDF lookup driven by stored uniform numbers (the first index whose
inclusive running sum exceeds ``u * total``), because multinomial's random stream
cannot be reproduced by anything but torch itself.  Sorting, running sums, the
mask ``probs_sum - probs_sort > p``, the renormalisation and the gathers are the
reference's own code.  Inputs are regenerated from their seeds by the tests; the
file stores the uniforms, thresholds and outputs.
"""

from __future__ import annotations

import argparse
import importlib.util
import types
from pathlib import Path

import numpy as np
import torch

CASES = [
    # name, rows, vocab, seed, logit scale, temperature
    ("flat", 12, 1000, 11, 1.0, 1.0),
    ("peaked", 12, 4096, 12, 4.0, 0.7),
    ("ragged", 7, 1537, 13, 2.5, 1.3),
    ("vocab", 3, 128256, 14, 3.0, 0.7),
]
TOP_PS = [0.0, 0.1, 0.5, 0.9, 0.95, 1.0]


def case_inputs(rows: int, vocab: int, seed: int, scale: float, temp: float):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(rows, vocab, generator=g) * scale
    u = torch.rand(rows, generator=g)
    p = torch.tensor([TOP_PS[i % len(TOP_PS)] for i in range(rows)])[:, None]
    probs = torch.softmax(logits / temp, dim=-1)
    return logits, probs, p, u


def load_reference(root: str):
    path = Path(root) / "cwm" / "fastgen" / "utils" / "sampling.py"
    spec = importlib.util.spec_from_file_location("ref_sampling_module", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference checkout")
    ap.add_argument("--out", default=str(Path(__file__).with_name("sampling_golden.npz")))
    args = ap.parse_args()
    mod = load_reference(args.reference)

    current_u: list[torch.Tensor] = []

    def multinomial(weights, num_samples=1, **_):
        assert num_samples == 1
        csum = torch.cumsum(weights, dim=-1)
        target = current_u[0].to(weights.dtype)[:, None] * csum[:, -1:]
        return (csum > target).to(torch.int8).argmax(dim=-1, keepdim=True)

    # the module sees torch with multinomial replaced; everything else is torch's
    proxy = types.SimpleNamespace(**{k: getattr(torch, k) for k in dir(torch) if not k.startswith("__")})
    proxy.multinomial = multinomial
    mod.torch = proxy

    out: dict[str, np.ndarray] = {}
    for name, rows, vocab, seed, scale, temp in CASES:
        _, probs, p, u = case_inputs(rows, vocab, seed, scale, temp)
        current_u[:] = [u]
        tok, prob = mod.sample(probs.clone())
        out[f"{name}_sample_tokens"] = tok.numpy().copy()
        out[f"{name}_sample_probs"] = prob.numpy().copy()
        tok, prob = mod.top_p(probs.clone(), p)
        out[f"{name}_top_p_tokens"] = tok.numpy().copy()
        out[f"{name}_top_p_probs"] = prob.numpy().copy()
        out[f"{name}_u"] = u.numpy().copy()
        out[f"{name}_p"] = p.numpy().copy()
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays")


if __name__ == "__main__":
    main()
