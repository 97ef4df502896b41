"""Token sampling: drop-ins for ``cwm/fastgen/utils/sampling.py`` and for
``FastGen._sample`` (``cwm/fastgen/generate.py:996-1014``).

``sample(probs)`` and ``top_p(probs, p)`` keep the reference's signatures and
return ``(next_tokens, next_tokens_prob)``; ``sample_logits`` is the fused form of
``_sample``: temperature softmax, optional nucleus truncation, renormalisation, the
draw and the log-probability in one launch over the fp32 logits.

The reference draws with ``torch.multinomial``.  Here the draw is an inverse-CDF
lookup with one uniform number per row, which the caller may pass (``uniforms``)
or which is taken from ``generator`` / torch's default CUDA generator.  Given the
same uniforms the result is a pure function of the inputs: it does not depend on
thread timing, so tensor-parallel ranks that share a generator state draw the
same tokens, as the reference's ranks do.
"""

from __future__ import annotations

import torch

from . import _lib
from .kernels import _on_device, _ptr, _require_cuda, _stream

MODE_GREEDY, MODE_INDEX_ORDER, MODE_TOP_P = 0, 1, 2


def _uniforms(rows: int, device: torch.device, uniforms: torch.Tensor | None,
              generator: torch.Generator | None) -> torch.Tensor:
    if uniforms is None:
        return torch.rand(rows, device=device, dtype=torch.float32, generator=generator)
    if uniforms.dtype != torch.float32 or uniforms.shape != (rows,) or not uniforms.is_contiguous():
        raise ValueError(f"uniforms must be a contiguous float32 tensor of shape ({rows},)")
    return uniforms


def _launch(x: torch.Tensor, is_logits: bool, temps: torch.Tensor | None,
            top_ps: torch.Tensor | None, uniforms: torch.Tensor | None, mode: int,
            want_kept: bool = False):
    if x.ndim != 2 or x.dtype != torch.float32:
        raise ValueError("expected a 2-D float32 tensor (rows, vocab)")
    if x.shape[1] > 1 and x.stride(1) != 1:
        raise ValueError("rows must have unit stride")
    rows, vocab = x.shape
    for name, t in (("temps", temps), ("top_ps", top_ps)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != rows
                              or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous float32 tensor with one value per row")
    _require_cuda("sample", x, temps, top_ps, uniforms)
    tokens = torch.empty(rows, dtype=torch.int64, device=x.device)
    probs = torch.empty(rows, dtype=torch.float32, device=x.device)
    kept = torch.empty(rows, dtype=torch.int32, device=x.device) if want_kept else None
    if rows == 0:
        return tokens, probs, kept
    with _on_device(x):
        code = _lib.load().cwm_sample(
            x.data_ptr(), int(is_logits), _ptr(temps), _ptr(top_ps), _ptr(uniforms), rows, vocab,
            x.stride(0) if rows > 1 else vocab, mode, tokens.data_ptr(), probs.data_ptr(),
            _ptr(kept), _stream(x),
        )
    _lib.check(code, "sample")
    return tokens, probs, kept


def sample(probs: torch.Tensor, *, uniforms: torch.Tensor | None = None,
           generator: torch.Generator | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``sample(probs)`` of ``sampling.py:6-18``: one draw per row of ``probs``
    ``(rows, vocab)``; returns the indices and their probabilities (as fractions
    of the row total)."""
    u = _uniforms(probs.shape[0], probs.device, uniforms, generator)
    tokens, p, _ = _launch(probs, False, None, None, u, MODE_INDEX_ORDER)
    return tokens, p


def top_p(probs: torch.Tensor, p: torch.Tensor | float, *, uniforms: torch.Tensor | None = None,
          generator: torch.Generator | None = None,
          return_kept: bool = False):
    """``top_p(probs, p)`` of ``sampling.py:21-45``: nucleus sampling.  ``p`` is a
    float or a tensor with one threshold per row (shape ``(rows, 1)`` in the
    reference).  Returns the indices and their renormalised probabilities (and,
    with ``return_kept``, how many entries survived the mask)."""
    rows = probs.shape[0]
    if not torch.is_tensor(p):
        p = torch.full((rows,), float(p), dtype=torch.float32, device=probs.device)
    p = p.reshape(-1).to(torch.float32).contiguous()
    u = _uniforms(rows, probs.device, uniforms, generator)
    tokens, pr, kept = _launch(probs, False, None, p, u, MODE_TOP_P, want_kept=return_kept)
    return (tokens, pr, kept) if return_kept else (tokens, pr)


def sample_logits(logits: torch.Tensor, temps: torch.Tensor | None, top_ps: torch.Tensor | None,
                  use_sampling: bool = True, *, uniforms: torch.Tensor | None = None,
                  generator: torch.Generator | None = None
                  ) -> tuple[torch.Tensor, torch.Tensor]:
    """``FastGen._sample`` (``generate.py:996-1014``) in one launch.

    ``logits``: fp32 ``(rows, vocab)``; ``temps``: fp32 ``(rows,)``; ``top_ps``:
    fp32 ``(rows,)``, or None when no lane uses top-p (the reference then draws in
    index order, otherwise in descending order of probability).  Returns
    ``(next_tokens int64, next_tokens_logprob fp32)``; with ``use_sampling`` False
    the tokens are the arg-maxima and the log-probabilities are zero.
    """
    if not use_sampling:
        tokens, _, _ = _launch(logits, True, None, None, None, MODE_GREEDY)
        return tokens, torch.zeros(logits.shape[0], dtype=logits.dtype, device=logits.device)
    u = _uniforms(logits.shape[0], logits.device, uniforms, generator)
    mode = MODE_INDEX_ORDER if top_ps is None else MODE_TOP_P
    tokens, p, _ = _launch(logits, True, temps, top_ps, u, mode)
    return tokens, torch.log(p)
