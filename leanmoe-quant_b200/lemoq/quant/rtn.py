"""Per-row, per-group symmetric RTN weight quantisation on the GPU.

Reference: src/lemoq/quant/rtn.py:38-99 (``quantize_rtn``).  Only the branch the canonical
decode path uses is built: 8-bit, symmetric, ``in_features % group_size == 0``.  The
arithmetic is the reference's, bit for bit: fp32 ``absmax/127`` scale (1.0 for an all-zero
group), ``round(w/scale)`` half-to-even with the fp32 scale, clamp to [-128, 127]; the
scale is stored as fp16 afterwards (src/lemoq/quant/linear.py:318-321).
"""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi


def qmax_for(bits: int, symmetric: bool = True) -> int:
    return (2 ** (bits - 1)) - 1 if symmetric else (2**bits) - 1


def quantize_w8(weight: Any, group_size: int = 128) -> tuple[Any, Any]:
    """``(..., in)`` fp16/fp32 CUDA tensor -> ``(codes int8 (..., in), scale fp16 (..., in/g))``."""
    if group_size <= 0:
        raise ValueError("group_size 必须 > 0")
    _cabi.require_cuda(weight, what="quantize_w8")
    w = weight if weight.dtype in (torch.float16, torch.float32) else weight.float()
    w = w.contiguous()
    in_features = int(w.shape[-1])
    rows = int(w.numel() // max(in_features, 1))
    codes = torch.empty(w.shape, dtype=torch.int8, device=w.device)
    scale = torch.empty((*w.shape[:-1], in_features // group_size if in_features % group_size == 0 else 0),
                        dtype=torch.float16, device=w.device)
    dt = _cabi.DTYPE_F16 if w.dtype == torch.float16 else _cabi.DTYPE_F32
    _cabi.call("lemoq_rtn_quantize_w8", _cabi.ptr(w), dt, rows, in_features, int(group_size), _cabi.ptr(codes),
               _cabi.ptr(scale), _cabi.current_stream(w.device))
    return codes, scale


def quantize_rtn(weight: Any, *, bits: int = 8, group_size: int = 128, symmetric: bool = True) -> dict[str, Any]:
    """Reference-shaped result dict for a 2-D weight.  ``codes`` is int8 and ``scale`` is the
    stored fp16 scale (the reference returns int32 codes and the fp32 scale; every decode-path
    consumer casts them to exactly these types)."""
    if weight.ndim != 2:
        raise ValueError("只支持 2-D 权重，得到 ndim=%d" % weight.ndim)
    if group_size <= 0:
        raise ValueError("group_size 必须 > 0")
    if bits != 8 or not symmetric:
        raise NotImplementedError(
            "只实现 8-bit 对称 RTN (only the symmetric 8-bit RTN of the canonical path is built); got bits=%r "
            "symmetric=%r" % (bits, symmetric))
    out_features, in_features = int(weight.shape[0]), int(weight.shape[1])
    if in_features % group_size != 0:
        raise NotImplementedError(
            "in_features=%d 不能被 group_size=%d 整除：本路径不补零" % (in_features, group_size))
    codes, scale = quantize_w8(weight, group_size)
    n_groups = in_features // group_size
    return {
        "codes": codes,
        "codes_padded": codes.reshape(out_features, n_groups, group_size),
        "scale": scale,
        "zero": torch.zeros_like(scale),
        "bits": bits,
        "group_size": group_size,
        "symmetric": True,
        "shape": (out_features, in_features),
        "n_groups": n_groups,
        "padded_in": in_features,
        "device": str(weight.device),
    }


def dequantize_rtn(q: dict[str, Any], dtype: Any = None) -> Any:
    """``codes * scale`` (host-side helper for the eager multi-token arm)."""
    out_features, in_features = q["shape"]
    codes = q["codes_padded"].reshape(out_features, q["n_groups"], q["group_size"]).float()
    w = (codes * q["scale"].float().reshape(out_features, q["n_groups"], 1)).reshape(out_features, in_features)
    return w.to(dtype) if dtype is not None else w
