"""CPU oracle for the FastGen attention hot path.  TEST INFRASTRUCTURE ONLY.

This package restates, in plain PyTorch fp32 on the CPU, what the reference
computes on its attention hot path (``cwm/fastgen/forward.py:601-656`` and the
helpers in ``cwm/fastgen/kernels``).  It exists to check the CUDA kernels and to
be timed as the CPU baseline.  Nothing in the product package may import it:
only the tests, the smoke check and the CPU-baseline leg of the benchmark do.

Pinning status
--------------
* ``ref_rope``, ``ref_rmsnorm``, ``ref_paged_memcpy``: pinned.  They are checked
  against outputs of the reference's own Triton kernels run under the Triton
  interpreter (fixtures in ``tests/golden``, produced by
  ``tests/golden/make_golden.py``).
* ``ref_paged_gqa_attention``: PARITY UNPINNED.  The reference delegates the
  arithmetic to ``xformers.ops.fmha.flash3.mha_fwd`` (xformers==0.0.31.post1,
  ``requirements.txt:25``), which is not vendored, and the reference ships no
  tests or golden vectors.  The restatement follows the published
  FlashAttention varlen/paged semantics and the reference call site
  (``forward.py:639-655``): bottom-right aligned causal mask, ``window_left``
  keys to the left of the diagonal, contiguous GQA head grouping.
"""

from .ref_ops import (  # noqa: F401
    ref_gqa_attention_layer,
    ref_paged_gqa_attention,
    ref_paged_memcpy,
    ref_prefill_splits,
    ref_rmsnorm,
    ref_rope,
    ref_rope_freqs,
)
