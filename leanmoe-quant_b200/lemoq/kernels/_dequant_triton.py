"""Compatibility name for ``lemoq.kernels._dequant_triton`` of the reference
(src/lemoq/kernels/_dequant_triton.py:155); the implementation is the CUDA kernel of
:mod:`lemoq.kernels.dequant_gemv`.  No Triton is involved."""

from lemoq.kernels.dequant_gemv import (  # noqa: F401
    DEQUANT_GEMM_CONFIGS,
    dequant_gemm_fused,
    fused_available,
    unavailable_reason,
    warm,
)
