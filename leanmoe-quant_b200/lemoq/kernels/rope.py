"""Fused half-split RoPE for the decode q/k rows (reference: src/lemoq/kernels/rope.py:160-203)."""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi

__all__ = ["apply_rotary_pos_emb_fused", "fused_rope_available", "rotate_half_reference", "warm"]


def _fused_rope_enabled() -> bool:
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("fused_rope")


def fused_rope_available() -> bool:
    return _cabi.available() and torch.cuda.is_available()


def rotate_half_reference(q: Any, k: Any, cos: Any, sin: Any, unsqueeze_dim: int = 1) -> tuple[Any, Any]:
    """The unfused chain (HF ``apply_rotary_pos_emb``): used for shapes the kernel does not take
    (prefill, batch > 1, CPU tensors)."""
    cos_u, sin_u = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)

    def rot(x):
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat((-x2, x1), dim=-1)

    return (q * cos_u) + (rot(q) * sin_u), (k * cos_u) + (rot(k) * sin_u)


def _decode_shape_guard(q: Any, k: Any, cos_u: Any, sin_u: Any) -> bool:
    if not (fused_rope_available() and q.is_cuda and k.is_cuda):
        return False
    if q.ndim != 4 or k.ndim != 4 or q.dtype != torch.float16:
        return False
    if any(t.dtype != q.dtype or t.device != q.device for t in (k, cos_u, sin_u)):
        return False
    if q.shape[0] != 1 or k.shape[0] != 1 or q.shape[2] != 1 or k.shape[2] != 1 or q.shape[3] != k.shape[3]:
        return False
    d = int(q.shape[3])
    if d % 2 != 0 or d < 2:
        return False
    if tuple(cos_u.shape) != (1, 1, 1, d) or tuple(sin_u.shape) != (1, 1, 1, d):
        return False
    if cos_u.stride(-1) != 1 or sin_u.stride(-1) != 1 or q.stride(3) != 1 or k.stride(3) != 1:
        return False
    return True


def apply_rotary_pos_emb_fused(q: Any, k: Any, cos: Any, sin: Any, position_ids: Any = None,
                               unsqueeze_dim: int = 1) -> tuple[Any, Any]:
    """One launch for q and k.  fp32 maths, one rounding to fp16.  Inputs that are not the decode
    shape ``(1, H, 1, D)`` fp16 on CUDA take the unfused chain instead."""
    cos_u, sin_u = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    if position_ids is not None or not _decode_shape_guard(q, k, cos_u, sin_u):
        return rotate_half_reference(q, k, cos, sin, unsqueeze_dim)
    d = int(q.shape[3])
    qo = torch.empty((1, int(q.shape[1]), 1, d), dtype=q.dtype, device=q.device)
    ko = torch.empty((1, int(k.shape[1]), 1, d), dtype=k.dtype, device=k.device)
    _cabi.call("lemoq_rope_qk", _cabi.ptr(q), int(q.stride(1)), int(q.shape[1]), _cabi.ptr(k), int(k.stride(1)),
               int(k.shape[1]), _cabi.ptr(cos_u), _cabi.ptr(sin_u), d, _cabi.ptr(qo), _cabi.ptr(ko),
               _cabi.current_stream(q.device))
    return qo, ko


def warm(*, heads: int = 16, kv_heads: int = 4, head_dim: int = 128, device: Any = None) -> None:
    if not fused_rope_available():
        return
    dev = device if device is not None else torch.device("cuda")
    q = torch.randn(1, heads, 1, head_dim, dtype=torch.float16, device=dev)
    k = torch.randn(1, kv_heads, 1, head_dim, dtype=torch.float16, device=dev)
    cos = torch.randn(1, 1, head_dim, dtype=torch.float16, device=dev)
    sin = torch.randn(1, 1, head_dim, dtype=torch.float16, device=dev)
    apply_rotary_pos_emb_fused(q, k, cos, sin)
    torch.cuda.synchronize(dev)
