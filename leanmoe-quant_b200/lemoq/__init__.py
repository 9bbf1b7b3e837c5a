"""lemoq: B200-native (sm_100a) kernels behind the LeanMoE-Quant kernel-op API.

The package mirrors the reference's ``lemoq`` module layout for the batch-1 OLMoE
decode path: ``lemoq.kernels`` (decode ops), ``lemoq.quant`` (W8 RTN + QuantLinear)
and ``lemoq.model`` (a transformers-free OLMoE module tree with the attribute names
the op API patches).  All device work is done by hand-written CUDA kernels reached
through the C-ABI library in ``csrc`` (see :mod:`lemoq._cabi`).
"""

__version__ = "0.1.0"
