"""B200 (sm_100a) kernels for the attention hot path of CWM's FastGen engine.

The public names mirror the reference's call sites so that they drop in:

* ``apply_rope``, ``paged_memcpy``, ``rmsnorm`` — ``cwm/fastgen/kernels``;
* ``mha_fwd`` — ``xformers.ops.fmha.flash3.mha_fwd`` as called by
  ``cwm/fastgen/forward.py:639-655``;
* ``AttnBias`` — the paged block-diagonal causal mask metadata of
  ``forward.py:12-14``;
* ``RawCache`` / ``ModelCache`` — ``cwm/fastgen/utils/cache.py``;
* ``gqa_attention`` — the GQA branch of ``forward.py:608-656`` in two launches;
* ``sampling`` — ``cwm/fastgen/utils/sampling.py`` and ``FastGen._sample``;
* ``hostcache`` (``Cache``, ``DynCache``), ``iset`` (``ISet``), ``engine`` (``Engine``) —
  ``cwm/fastgen/utils/cache.py:172-483``, ``utils/iset.py``, ``generate.py``;
* ``decoder`` — the GQA-only ``prefill`` / ``decode`` passes of ``forward.py:824-961``.

Everything runs through ``libcwm_b200.so``; there is no CPU or Triton fallback.
"""

from . import sampling
from .attention import mha_fwd, qkv_rope_kv_write, rope_kv_write, silu_mul, workspace_for
from .attn_bias import AttnBias, PagedBlockDiagonalCausalWithOffsetPaddedKeysMask
from .cache import ModelCache, RawCache
from .kernels import add_rmsnorm, apply_rope, paged_memcpy, rmsnorm
from .layer import gqa_attention, prefill_chunks, rope_freqs, window_size_left

__all__ = [
    "AttnBias",
    "ModelCache",
    "PagedBlockDiagonalCausalWithOffsetPaddedKeysMask",
    "RawCache",
    "add_rmsnorm",
    "apply_rope",
    "gqa_attention",
    "mha_fwd",
    "paged_memcpy",
    "prefill_chunks",
    "rmsnorm",
    "rope_freqs",
    "qkv_rope_kv_write",
    "rope_kv_write",
    "sampling",
    "silu_mul",
    "window_size_left",
    "workspace_for",
]
