"""Fused RMSNorm (reference: src/lemoq/kernels/rmsnorm.py:102-242).

``y = (x * rsqrt(mean(x^2) + eps)).to(fp16) * weight`` with the HF rounding chain: the
normalised value is rounded to fp16 before the fp16 multiply by the weight.
"""

from __future__ import annotations

import types
from typing import Any

import torch

from lemoq import _cabi

__all__ = ["RMSNORM_IMPL_DEFAULT", "RMSNORM_IMPLS", "fused_available", "unavailable_reason", "rms_norm_fused",
           "warm", "replace_rms_norms", "restore_rms_norms", "rms_norms_replaced"]

RMSNORM_IMPL_DEFAULT = "fused"
RMSNORM_IMPLS = ("fused", "hf")


def fused_available() -> bool:
    return _cabi.available() and torch.cuda.is_available()


def unavailable_reason() -> str | None:
    if not _cabi.available():
        return _cabi.unavailable_reason()
    if not torch.cuda.is_available():
        return "本机没有可用的 CUDA 设备 (no CUDA device)"
    return None


def rms_norm_fused(x: Any, weight: Any, eps: float, *, out_dtype: Any = None, config: dict[str, Any] | None = None) -> Any:
    """``x (..., H)`` fp16 contiguous, ``weight (H,)`` fp16 -> same shape.  Contract violations
    raise (ValueError / NotImplementedError), they never compute something else."""
    if x.dim() < 1:
        raise ValueError("x 至少要有一维")
    if not x.is_contiguous():
        raise ValueError("x 必须是连续的 (must be contiguous)")
    if not weight.is_contiguous():
        raise ValueError("weight 必须是连续的")
    if x.dtype != torch.float16:
        raise NotImplementedError("x 只支持 fp16，得到 %s" % x.dtype)
    if weight.dtype != torch.float16:
        raise NotImplementedError("weight 只支持 fp16，得到 %s" % weight.dtype)
    h = int(x.shape[-1])
    if int(weight.numel()) != h or weight.dim() != 1:
        raise ValueError("weight 必须是 (H,) 且 H=%d，得到 %r" % (h, tuple(weight.shape)))
    if h & (h - 1) != 0:
        raise NotImplementedError("H 必须是 2 的幂，得到 %d" % h)
    if h > 8192:
        raise NotImplementedError("H=%d 超过本 kernel 的块上限 8192" % h)
    if out_dtype is not None and out_dtype != torch.float16:
        raise NotImplementedError("out_dtype 只支持 fp16")
    _cabi.require_cuda(x, weight, what="rms_norm_fused")
    y = torch.empty_like(x)
    rows = int(x.numel()) // h
    _cabi.call("lemoq_rms_norm", _cabi.ptr(x), _cabi.ptr(weight), _cabi.ptr(y), rows, h, float(eps),
               _cabi.current_stream(x.device))
    return y


def warm(x: Any, weight: Any, eps: float, **kwargs: Any) -> None:
    rms_norm_fused(x, weight, eps, **kwargs)


def _fused_norm_forward(self: Any, hidden_states: Any) -> Any:
    x = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
    return rms_norm_fused(x, self.weight, float(self.variance_epsilon), out_dtype=x.dtype)


def replace_rms_norms(model: Any, impl: str = RMSNORM_IMPL_DEFAULT) -> int:
    """Switch every ``OlmoeRMSNorm`` instance to ``impl`` (instance-level, reversible)."""
    if impl not in RMSNORM_IMPLS:
        raise ValueError("未知 rmsnorm 实现 %r；可用 %s" % (impl, list(RMSNORM_IMPLS)))
    n = 0
    for module in model.modules():
        if type(module).__name__ != "OlmoeRMSNorm" or not hasattr(module, "variance_epsilon"):
            continue
        if not hasattr(module, "_lemoq_original_norm"):
            module._lemoq_original_norm = module.forward
        module.forward = (module._lemoq_original_norm if impl == "hf"
                          else types.MethodType(_fused_norm_forward, module))
        n += 1
    return n


def restore_rms_norms(model: Any) -> int:
    n = 0
    for module in model.modules():
        if hasattr(module, "_lemoq_original_norm"):
            module.forward = module._lemoq_original_norm
            del module._lemoq_original_norm
            n += 1
    return n


def rms_norms_replaced(model: Any) -> int:
    return sum(1 for m in model.modules()
               if hasattr(m, "_lemoq_original_norm") and m.forward is not m._lemoq_original_norm)
