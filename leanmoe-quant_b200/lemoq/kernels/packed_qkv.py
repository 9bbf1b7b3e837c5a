"""Packed q/k/v projection: one W8 GEMV over the concatenated ``[q; k; v]`` rows
(reference: src/lemoq/kernels/packed_qkv.py).  Row-local reduction order, so the packed result is
bit-identical to three separate calls."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

SWITCH = "LEMOQ_PACKED_QKV"


def packed_qkv_enabled() -> bool:
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("packed_qkv")


def packed_qkv_applicable(attn: Any, quantized: bool) -> bool:
    """Both preconditions: ``attn == "kernel"`` and the cell is quantised; otherwise a no-op."""
    return str(attn) == "kernel" and bool(quantized)


def _attention_modules(model: Any) -> list[Any]:
    from lemoq.kernels.attn_decode import _attention_modules as _select

    return list(_select(model))


@dataclass
class PackedQKV:
    packed: Any
    scale: Any
    in_features: int
    out_features: int
    group_size: int

    def project(self, x: Any) -> tuple[Any, Any, Any]:
        from lemoq.kernels.dequant_gemv import dequant_gemm_fused

        flat = x.reshape(-1, self.in_features)
        if not flat.is_contiguous():
            flat = flat.contiguous()
        y = dequant_gemm_fused(flat, self.packed, self.scale, None, group_size=self.group_size, bits=8, symmetric=True,
                               out_dtype=x.dtype)
        y = y.reshape(*x.shape[:-1], 3, self.out_features)
        return y[..., 0, :], y[..., 1, :], y[..., 2, :]

    def combined(self, x: Any) -> Any:
        return torch.cat(self.project(x), dim=-1)


def _validate(layer: Any, q: Any, k: Any, v: Any) -> None:
    from lemoq.quant.linear import QuantLinear

    for role, module in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
        if not isinstance(module, QuantLinear):
            raise ValueError("packed q/k/v 需要已量化的 %s（layer=%r 得到 %s）" % (role, layer, type(module).__name__))
        if int(module.weight_bits) != 8:
            raise NotImplementedError("packed q/k/v 只支持 w8（%s 是 %d-bit）" % (role, int(module.weight_bits)))
        if not bool(module.spec.symmetric) or module.zero is not None:
            raise NotImplementedError("packed q/k/v 只支持对称量化（%s）" % role)
        if module.bias is not None:
            raise NotImplementedError("packed q/k/v 不支持带 bias 的投影（%s）" % role)
    shape = {(int(m.in_features), int(m.out_features), int(m.group_size), int(m.padded_in), int(m.n_groups))
             for m in (q, k, v)}
    if len(shape) != 1:
        raise ValueError("packed q/k/v 要求三个投影的 (in, out, group, padded_in, n_groups) 完全一致，得到 %r" % (sorted(shape),))


def install_packed_qkv(model: Any) -> int:
    """Build the concatenated buffers on every attention module (after quantisation, before capture)."""
    installed = 0
    for module in _attention_modules(model):
        q, k, v = (getattr(module, n, None) for n in ("q_proj", "k_proj", "v_proj"))
        _validate(getattr(module, "layer_idx", "?"), q, k, v)
        module._lemoq_packed_qkv = PackedQKV(
            packed=torch.cat((q.packed, k.packed, v.packed), dim=0).contiguous(),
            scale=torch.cat((q.scale, k.scale, v.scale), dim=0).contiguous(),
            in_features=int(q.in_features), out_features=int(q.out_features), group_size=int(q.group_size))
        installed += 1
    if not installed:
        raise RuntimeError("没有找到任何 OLMoE attention 模块 (no OLMoE attention module found)")
    return installed


def packed_qkv_installed(model: Any) -> int:
    return sum(1 for m in _attention_modules(model) if getattr(m, "_lemoq_packed_qkv", None) is not None)


def remove_packed_qkv(model: Any) -> int:
    removed = 0
    for module in _attention_modules(model):
        if getattr(module, "_lemoq_packed_qkv", None) is not None:
            delattr(module, "_lemoq_packed_qkv")
            removed += 1
    return removed
