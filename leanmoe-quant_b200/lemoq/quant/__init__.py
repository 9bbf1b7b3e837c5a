"""W8 weight quantisation (reference: ``lemoq.quant``; only the symmetric 8-bit RTN of the
canonical decode path is built)."""

from lemoq.quant.rtn import dequantize_rtn, qmax_for, quantize_rtn  # noqa: F401
