"""Packed q/k/v projection: the three W8 projections of an attention module as ONE GEMV over their rows
stacked ``[q; k; v]`` (the interface of the reference's src/lemoq/kernels/packed_qkv.py:50-164).

The GEMV kernel reduces every output row on its own, in an order that does not depend on how many rows
the call has, so the stacked call returns the very bits three separate calls return
(tests/test_gpu_ops.py checks that).  The stacked buffers are built once, after quantisation and before
any graph capture; the decode step hands their pointers to the native step engine.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

SWITCH = "LEMOQ_PACKED_QKV"
_ATTR = "_lemoq_packed_qkv"
_ROLES = ("q_proj", "k_proj", "v_proj")


def packed_qkv_enabled() -> bool:
    """State of the ``packed_qkv`` fusion switch (read when the buffers are built)."""
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("packed_qkv")


def packed_qkv_applicable(attn: Any, quantized: bool) -> bool:
    """The stacked projection exists only for the kernel attention on a quantised cell; everywhere else the
    switch is a no-op (never a refusal)."""
    return bool(quantized) and str(attn) == "kernel"


def _attention_modules(model: Any) -> list[Any]:
    from lemoq.kernels.attn_decode import _attention_modules as select

    return list(select(model))


def _geometry(module: Any) -> tuple[int, int, int, int, int]:
    return tuple(int(getattr(module, name)) for name in ("in_features", "out_features", "group_size", "padded_in", "n_groups"))


def _check_projections(layer: Any, projections: dict[str, Any]) -> None:
    """What the stacked form needs of each projection, one rule per line: (holds?, error type, message)."""
    from lemoq.quant.linear import QuantLinear

    for role, m in projections.items():
        quantised = isinstance(m, QuantLinear)
        rules = (
            (quantised, ValueError, "packed q/k/v 需要已量化的 %s（layer=%r 得到 %s）" % (role, layer, type(m).__name__)),
            (quantised and int(m.weight_bits) == 8, NotImplementedError,
             "packed q/k/v 只支持 w8（%s 是 %s-bit）" % (role, getattr(m, "weight_bits", "?"))),
            (quantised and bool(m.spec.symmetric) and m.zero is None, NotImplementedError, "packed q/k/v 只支持对称量化（%s）" % role),
            (quantised and m.bias is None, NotImplementedError, "packed q/k/v 不支持带 bias 的投影（%s）" % role),
        )
        for holds, error, message in rules:
            if not holds:
                raise error(message)
    shapes = sorted({_geometry(m) for m in projections.values()})
    if len(shapes) > 1:
        raise ValueError("packed q/k/v 要求三个投影的 (in, out, group, padded_in, n_groups) 完全一致，得到 %r" % (shapes,))


@dataclass
class PackedQKV:
    """Stacked int8 codes ``(3 * out, in)`` and fp16 group scales ``(3 * out, in / group)`` of one attention module."""

    packed: Any
    scale: Any
    in_features: int
    out_features: int
    group_size: int

    @classmethod
    def stack(cls, q: Any, k: Any, v: Any) -> "PackedQKV":
        parts = (q, k, v)
        return cls(packed=torch.cat([m.packed for m in parts]).contiguous(), scale=torch.cat([m.scale for m in parts]).contiguous(),
                   in_features=int(q.in_features), out_features=int(q.out_features), group_size=int(q.group_size))

    def combined(self, x: Any) -> Any:
        """``[..., 3 * out]``: q, k and v of every row of ``x`` side by side (one kernel call)."""
        from lemoq.kernels.dequant_gemv import dequant_gemm_fused

        rows = x.reshape(-1, self.in_features).contiguous()
        y = dequant_gemm_fused(rows, self.packed, self.scale, None, group_size=self.group_size, bits=8, symmetric=True,
                               out_dtype=x.dtype)
        return y.reshape(*x.shape[:-1], 3 * self.out_features)

    def project(self, x: Any) -> tuple[Any, Any, Any]:
        """``(q, k, v)`` as views of the one result."""
        q, k, v = self.combined(x).split(self.out_features, dim=-1)
        return q, k, v


def install_packed_qkv(model: Any) -> int:
    """Attach a :class:`PackedQKV` to every OLMoE attention module; returns how many.  Call it after quantisation and
    before capture (it allocates)."""
    modules = _attention_modules(model)
    if not modules:
        raise RuntimeError("没有找到任何 OLMoE attention 模块 (no OLMoE attention module found)")
    for module in modules:
        projections = {role: getattr(module, role, None) for role in _ROLES}
        _check_projections(getattr(module, "layer_idx", "?"), projections)
        setattr(module, _ATTR, PackedQKV.stack(*projections.values()))
    return len(modules)


def packed_qkv_installed(model: Any) -> int:
    return sum(getattr(m, _ATTR, None) is not None for m in _attention_modules(model))


def remove_packed_qkv(model: Any) -> int:
    carrying = [m for m in _attention_modules(model) if getattr(m, _ATTR, None) is not None]
    for module in carrying:
        delattr(module, _ATTR)
    return len(carrying)
