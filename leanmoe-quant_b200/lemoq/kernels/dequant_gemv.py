"""Dense W8 dequant GEMV (reference: src/lemoq/kernels/_dequant_triton.py:155-293).

``y = x @ dequant(qweight, scale).T`` with the int8 codes dequantised in registers.  Only the
symmetric 8-bit format of the canonical decode path is built; other formats raise
``NotImplementedError`` like any unsupported variant in the reference.
"""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi

__all__ = ["DEQUANT_GEMM_CONFIGS", "dequant_gemm_fused", "fused_available", "unavailable_reason", "warm"]

# Tile description of the CUDA kernel (informational: it is not tunable from Python).
# One warp streams two weight rows; a row is read as 128-bit words, 16 codes per lane.
DEQUANT_GEMM_CONFIGS: dict[str, dict[str, int]] = {
    "dequant_gemm": {"ROWS_PER_WARP": 2, "BYTES_PER_LANE": 16, "num_warps": 8},
}


def fused_available() -> bool:
    """Whether the fused arm can run here (library built and a CUDA device present)."""
    return _cabi.available() and torch.cuda.is_available()


def unavailable_reason() -> str | None:
    if not _cabi.available():
        return _cabi.unavailable_reason()
    if not torch.cuda.is_available():
        return "本机没有可用的 CUDA 设备 (no CUDA device)"
    return None


def dequant_gemm_fused(x: Any, qweight: Any, scale: Any, zero: Any = None, *, group_size: int,
                       bits: int | None = None, symmetric: bool = True, out_dtype: Any = None,
                       config: dict[str, Any] | None = None, mxfp4: bool = False) -> Any:
    """``x (M, K)`` fp16, ``qweight (N, K)`` int8, ``scale (N, K/g)`` fp16 -> ``(M, N)``.

    ``out_dtype=None`` returns fp32 like the reference.  All tensors must be contiguous.
    """
    if x.dim() != 2:
        raise ValueError("x 必须是 (M, K) 二维，得到 %r" % (tuple(x.shape),))
    if qweight.dim() != 2:
        raise ValueError("qweight 必须是 (N, P) 二维，得到 %r" % (tuple(qweight.shape),))
    if scale.dim() != 2:
        raise ValueError("scale 必须是 (N, n_groups) 二维，得到 %r" % (tuple(scale.shape),))
    if mxfp4 or not symmetric or zero is not None:
        raise NotImplementedError("只实现对称 w8 (only symmetric w8 is built on this path)")
    if bits is None:
        bits = 4 if qweight.dtype == torch.uint8 else 8
    if int(bits) != 8:
        raise NotImplementedError("fused dequant-GEMV 只实现 8-bit，得到 %d" % int(bits))
    m, k = int(x.shape[0]), int(x.shape[1])
    n, packed_in = int(qweight.shape[0]), int(qweight.shape[1])
    n_groups = int(scale.shape[1])
    if int(scale.shape[0]) != n:
        raise ValueError("scale 的行数 %d 与 qweight 的 %d 不一致" % (int(scale.shape[0]), n))
    if packed_in != n_groups * int(group_size):
        raise ValueError("qweight 的第二维 %d 与 n_groups*group_size=%d 不一致" % (packed_in, n_groups * int(group_size)))
    if k != packed_in:
        raise NotImplementedError("K=%d != padded_in=%d：本路径不补零 (no zero padding)" % (k, packed_in))
    if qweight.dtype != torch.int8:
        raise ValueError("8-bit 对称 qweight 应是 int8，得到 %s" % qweight.dtype)
    if scale.dtype != torch.float16:
        raise NotImplementedError("scale 只支持 fp16，得到 %s" % scale.dtype)
    if x.dtype != torch.float16:
        raise NotImplementedError("x 只支持 fp16，得到 %s" % x.dtype)
    out_dtype = torch.float32 if out_dtype is None else out_dtype
    if out_dtype not in (torch.float32, torch.float16):
        raise NotImplementedError("out_dtype 只支持 fp32/fp16，得到 %s" % out_dtype)
    for name, tensor in (("x", x), ("qweight", qweight), ("scale", scale)):
        if not tensor.is_contiguous():
            raise ValueError("%s 必须是连续的 (must be contiguous)" % name)
    _cabi.require_cuda(x, qweight, scale, what="dequant_gemm_fused")
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _cabi.call("lemoq_dequant_gemv_w8", _cabi.ptr(x), m, _cabi.ptr(qweight), _cabi.ptr(scale), n, k, int(group_size),
               _cabi.ptr(y), _cabi.DTYPE_F16 if out_dtype == torch.float16 else _cabi.DTYPE_F32,
               _cabi.current_stream(x.device))
    return y


def warm(x: Any, qweight: Any, scale: Any, zero: Any = None, **kwargs: Any) -> None:
    """One real launch before capture (the kernels are precompiled; kept for API parity)."""
    dequant_gemm_fused(x, qweight, scale, zero, **kwargs)
