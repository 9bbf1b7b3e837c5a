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


_MAX_WIDTH = 8192  # one block normalises one row held in registers


def rms_norm_fused(x: Any, weight: Any, eps: float, *, out_dtype: Any = None, config: dict[str, Any] | None = None) -> Any:
    """``x (..., H)`` fp16 contiguous, ``weight (H,)`` fp16 -> the same shape.  A call outside the contract raises
    (``ValueError`` for a wrong shape or layout, ``NotImplementedError`` for a dtype or width the kernel does not
    take); it never computes something else."""
    if x.dim() < 1:
        raise ValueError("x 至少要有一维 (at least one dimension)")
    width = int(x.shape[-1])
    refusals = (
        (x.is_contiguous() and weight.is_contiguous(), ValueError, "x 和 weight 必须是连续的 (must be contiguous)"),
        (x.dtype == torch.float16 and weight.dtype == torch.float16, NotImplementedError,
         "x / weight 只支持 fp16 (got %s / %s)" % (x.dtype, weight.dtype)),
        (tuple(weight.shape) == (width,), ValueError, "weight 必须是 (H,) with H=%d, got %r" % (width, tuple(weight.shape))),
        (width & (width - 1) == 0, NotImplementedError, "H 必须是 2 的幂 (power of two), got %d" % width),
        (width <= _MAX_WIDTH, NotImplementedError, "H=%d 超过本 kernel 的块上限 %d" % (width, _MAX_WIDTH)),
        (out_dtype in (None, torch.float16), NotImplementedError, "out_dtype 只支持 fp16"),
    )
    for ok, error, text in refusals:
        if not ok:
            raise error(text)
    _cabi.require_cuda(x, weight, what="rms_norm_fused")
    y = torch.empty_like(x)
    _cabi.call("lemoq_rms_norm", _cabi.ptr(x), _cabi.ptr(weight), _cabi.ptr(y), x.numel() // width, width, float(eps),
               _cabi.current_stream(x.device))
    return y


def warm(x: Any, weight: Any, eps: float, **kwargs: Any) -> None:
    """Kept for the reference's call sites: the kernel is precompiled, one call is all there is to warm."""
    rms_norm_fused(x, weight, eps, **kwargs)


def _fused_norm_forward(self: Any, hidden_states: Any) -> Any:
    return rms_norm_fused(hidden_states.contiguous(), self.weight, float(self.variance_epsilon), out_dtype=hidden_states.dtype)


_KEPT = "_lemoq_original_norm"


def _olmoe_norms(model: Any) -> list[Any]:
    return [m for m in model.modules() if type(m).__name__ == "OlmoeRMSNorm" and hasattr(m, "variance_epsilon")]


def replace_rms_norms(model: Any, impl: str = RMSNORM_IMPL_DEFAULT) -> int:
    """Point every ``OlmoeRMSNorm`` instance at ``impl`` ("fused": the kernel, "hf": the module's own forward).  The
    module's own forward is kept on the instance, so the switch goes both ways."""
    if impl not in RMSNORM_IMPLS:
        raise ValueError("未知 rmsnorm 实现 %r (unknown impl); have %s" % (impl, list(RMSNORM_IMPLS)))
    norms = _olmoe_norms(model)
    for norm in norms:
        own = norm.__dict__.setdefault(_KEPT, norm.forward)
        norm.forward = own if impl == "hf" else types.MethodType(_fused_norm_forward, norm)
    return len(norms)


def restore_rms_norms(model: Any) -> int:
    kept = [m for m in model.modules() if hasattr(m, _KEPT)]
    for norm in kept:
        norm.forward = norm.__dict__.pop(_KEPT)
    return len(kept)


def rms_norms_replaced(model: Any) -> int:
    return sum(hasattr(m, _KEPT) and m.forward is not getattr(m, _KEPT) for m in model.modules())
