"""Grouped MoE decode on W8 expert weights (reference: src/lemoq/kernels/moe_grouped_quant.py).

The stacked expert tensors are RTN-quantised per row and per group of 128 along K; the kernels
read int8 codes + fp16 scales and dequantise in registers, so the fp16 weights never exist in HBM.
"""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Any

import torch

from lemoq import _cabi
from lemoq.kernels.moe_grouped import _MAX_OFFSET, PARITY_GATE, launch_plan, merged_config  # noqa: F401

__all__ = ["QuantFusedExperts", "dequantize_fused_experts", "grouped_moe_forward_quant", "quant_launch_plan",
           "quantize_fused_experts", "quantized_grouped_available", "static_moe_forward_grouped_quant"]


@dataclass
class QuantFusedExperts:
    """``packed_gate_up (E, 2F, H)`` int8, ``scale_gate_up (E, 2F, H/g)`` fp16,
    ``packed_down (E, H, F)`` int8, ``scale_down (E, H, F/g)`` fp16; gate rows ``[0, F)``, up rows
    ``[F, 2F)``; groups run along the last (K) dim."""

    packed_gate_up: Any
    scale_gate_up: Any
    packed_down: Any
    scale_down: Any
    bits: int
    group_size: int

    @property
    def num_experts(self) -> int:
        return int(self.packed_gate_up.shape[0])

    @property
    def ffn(self) -> int:
        return int(self.packed_gate_up.shape[1]) // 2

    @property
    def hidden(self) -> int:
        return int(self.packed_gate_up.shape[-1]) * (8 // int(self.bits))

    def nbytes(self) -> int:
        return sum(int(t.numel()) * int(t.element_size())
                   for t in (self.packed_gate_up, self.scale_gate_up, self.packed_down, self.scale_down))

    def to(self, device: Any = None, dtype: Any = None) -> "QuantFusedExperts":
        """Device moves only: codes stay int8 and scales stay fp16."""
        if isinstance(device, torch.dtype):
            device, dtype = None, device
        if dtype is not None:
            raise ValueError("QuantFusedExperts 不支持 dtype 转换 (codes are int8, scales fp16); got dtype=%r" % (dtype,))
        if device is None:
            return self
        return QuantFusedExperts(*(t.to(device=device).contiguous() for t in (
            self.packed_gate_up, self.scale_gate_up, self.packed_down, self.scale_down)),
            bits=self.bits, group_size=self.group_size)

    # dequantisation: eager multi-token (prefill) arm only, never on the decode path
    def _dequant_2d(self, codes: Any, scale: Any, dtype: Any) -> Any:
        rows, k = int(codes.shape[0]), int(codes.shape[1])
        ng = k // self.group_size
        w = (codes.reshape(rows, ng, self.group_size).float() * scale.reshape(rows, ng, 1).float()).reshape(rows, k)
        return w.to(dtype) if dtype is not None else w

    def dequant_gate_up_expert(self, index: int, dtype: Any = None) -> Any:
        return self._dequant_2d(self.packed_gate_up[index], self.scale_gate_up[index], dtype)

    def dequant_down_expert(self, index: int, dtype: Any = None) -> Any:
        return self._dequant_2d(self.packed_down[index], self.scale_down[index], dtype)

    def dequant_gate_up(self, dtype: Any = None) -> Any:
        e, rows, k = (int(v) for v in self.packed_gate_up.shape)
        return self._dequant_2d(self.packed_gate_up.reshape(e * rows, k), self.scale_gate_up.reshape(e * rows, -1),
                                dtype).reshape(e, rows, k)

    def dequant_down(self, dtype: Any = None) -> Any:
        e, rows, k = (int(v) for v in self.packed_down.shape)
        return self._dequant_2d(self.packed_down.reshape(e * rows, k), self.scale_down.reshape(e * rows, -1),
                                dtype).reshape(e, rows, k)


def quantize_fused_experts(fused: Any, *, bits: int = 8, group_size: int = 128) -> QuantFusedExperts:
    """RTN on the stacked ``(E, 2F, H)`` / ``(E, H, F)`` tensors (row-local, hence bit-identical to
    quantising each expert alone).  Runs the CUDA quantiser."""
    from lemoq.quant.rtn import quantize_w8

    if bits != 8:
        raise NotImplementedError("量化 grouped 路径只实现 8-bit (canonical W8A16)，得到 %r" % (bits,))
    if group_size <= 0:
        raise ValueError("group_size 必须 > 0")
    hidden, ffn = int(fused.gate_up.shape[2]), int(fused.down.shape[2])
    for name, dim in (("hidden", hidden), ("ffn", ffn)):
        if dim % group_size != 0:
            raise NotImplementedError("%s=%d 不能被 group_size=%d 整除：量化 grouped 路径不补零" % (name, dim, group_size))
    cg, sg = quantize_w8(fused.gate_up, group_size)
    cd, sd = quantize_w8(fused.down, group_size)
    return QuantFusedExperts(cg.contiguous(), sg.contiguous(), cd.contiguous(), sd.contiguous(), int(bits), int(group_size))


def dequantize_fused_experts(q: QuantFusedExperts, dtype: Any = None) -> Any:
    from lemoq.kernels.moe_static import FusedExperts

    return FusedExperts(gate_up=q.dequant_gate_up(dtype=dtype), down=q.dequant_down(dtype=dtype))


def quantized_grouped_available() -> bool:
    return _cabi.available() and torch.cuda.is_available()


class _ShapeShim:
    def __init__(self, shape: tuple) -> None:
        self.shape = tuple(shape)


def quant_launch_plan(q: QuantFusedExperts, *, top_k: int, config: dict[str, Any] | None = None,
                      for_kernel: bool = True) -> dict[str, Any]:
    """Grid/buffer shapes plus the quantisation-specific contract checks (violations raise)."""
    e, ffn, hidden = int(q.packed_gate_up.shape[0]), int(q.packed_gate_up.shape[1]) // 2, q.hidden
    plan = launch_plan(SimpleNamespace(gate_up=_ShapeShim((e, 2 * ffn, hidden)), down=_ShapeShim((e, hidden, ffn))),
                       top_k=top_k, config=config)
    if int(q.bits) != 8:
        raise NotImplementedError("量化 grouped 路径只实现 8-bit，得到 %d" % int(q.bits))
    for name, tensor in (("packed_gate_up", q.packed_gate_up), ("scale_gate_up", q.scale_gate_up),
                         ("packed_down", q.packed_down), ("scale_down", q.scale_down)):
        if not tensor.is_contiguous():
            raise ValueError("%s 必须连续 (must be contiguous)" % name)
        if int(tensor.numel()) >= _MAX_OFFSET:
            raise ValueError("%s 的元素数超过 int32 偏移上限" % name)
    group = int(q.group_size)
    for name, dim in (("hidden", plan["hidden"]), ("ffn", plan["ffn"])):
        if dim % group != 0:
            raise ValueError("%s=%d 不能被 group_size=%d 整除" % (name, dim, group))
    if for_kernel and group % 16 != 0:
        raise ValueError("group_size=%d 必须是 16 的倍数：一个 lane 的 16 个 code (BLOCK_K 片) 共用一个 scale" % group)
    plan["quant"] = {"bits": int(q.bits), "group_size": group, "for_kernel": bool(for_kernel),
                     "packed_gate_up_bytes": int(q.packed_gate_up.numel()),
                     "scale_gate_up_bytes": int(q.scale_gate_up.numel()) * int(q.scale_gate_up.element_size())}
    return plan


def grouped_moe_forward_quant(x: Any, q: QuantFusedExperts, ids: Any, top_w: Any, *,
                              config: dict[str, Any] | None = None, backend: str = "auto") -> Any:
    """``(H,)`` hidden state + ``(K,)`` expert ids + ``(K,)`` routing weights -> ``(H,)`` fp16."""
    if backend == "oracle":
        raise RuntimeError("backend='oracle' is not part of this package (the CPU oracle is test infrastructure)")
    if backend not in ("auto", "cuda", "triton"):
        raise ValueError("unknown backend %r" % (backend,))
    if q.scale_gate_up.dtype != torch.float16:
        raise NotImplementedError("量化 grouped kernel 只支持 fp16 scale；得到 scale_gate_up.dtype=%s"
                                  % str(q.scale_gate_up.dtype).replace("torch.", ""))
    if not quantized_grouped_available():
        raise RuntimeError("量化 grouped kernels 不可用: %s" % (_cabi.unavailable_reason() or "no CUDA device"))
    dt = q.scale_gate_up.dtype
    xf = x.reshape(-1).contiguous()
    if xf.dtype != dt:
        xf = xf.to(dt)
    idx = ids.reshape(-1).contiguous()
    if idx.dtype != torch.int64:
        idx = idx.to(torch.int64)
    wsum = top_w.reshape(-1).contiguous()
    if wsum.dtype != dt:
        wsum = wsum.to(dt)
    top_k = int(idx.numel())
    plan = quant_launch_plan(q, top_k=top_k, config=config, for_kernel=True)
    hidden, ffn = int(plan["hidden"]), int(plan["ffn"])
    if int(xf.numel()) != hidden:
        raise ValueError("grouped_moe_forward_quant 只处理单 token：x 有 %d 个元素，hidden 是 %d" % (int(xf.numel()), hidden))
    if int(wsum.numel()) != top_k:
        raise ValueError("top_w 的长度 %d 与槽位数 %d 不符" % (int(wsum.numel()), top_k))
    _cabi.require_cuda(xf, q.packed_gate_up, idx, wsum, what="grouped_moe_forward_quant")
    act = torch.empty((top_k, ffn), dtype=dt, device=xf.device)
    out = torch.empty((hidden,), dtype=dt, device=xf.device)
    _cabi.call("lemoq_moe_grouped_w8", _cabi.ptr(xf), _cabi.ptr(q.packed_gate_up), _cabi.ptr(q.scale_gate_up),
               _cabi.ptr(q.packed_down), _cabi.ptr(q.scale_down), _cabi.ptr(idx), _cabi.ptr(wsum), 1, top_k,
               q.num_experts, hidden, ffn, int(q.group_size), _cabi.ptr(act), _cabi.ptr(out), None,
               _cabi.current_stream(xf.device))
    return out


def grouped_moe_forward_quant_tokens(x: Any, q: QuantFusedExperts, ids: Any, top_w: Any) -> Any:
    """Batched form for the grouped-GEMV microbenchmark: ``x (T, H)``, ``ids/top_w (T, K)`` ->
    ``(T, H)``.  Each token is an independent one-token problem."""
    t, hidden = int(x.shape[0]), int(x.shape[1])
    k = int(ids.shape[1])
    dt = q.scale_gate_up.dtype
    _cabi.require_cuda(x, ids, top_w, what="grouped_moe_forward_quant_tokens")
    xf, idx, wsum = x.to(dt).contiguous(), ids.to(torch.int64).contiguous(), top_w.to(dt).contiguous()
    act = torch.empty((t, k, q.ffn), dtype=dt, device=x.device)
    out = torch.empty((t, hidden), dtype=dt, device=x.device)
    _cabi.call("lemoq_moe_grouped_w8", _cabi.ptr(xf), _cabi.ptr(q.packed_gate_up), _cabi.ptr(q.scale_gate_up),
               _cabi.ptr(q.packed_down), _cabi.ptr(q.scale_down), _cabi.ptr(idx), _cabi.ptr(wsum), t, k,
               q.num_experts, hidden, q.ffn, int(q.group_size), _cabi.ptr(act), _cabi.ptr(out), None,
               _cabi.current_stream(x.device))
    return out


def static_moe_forward_grouped_quant(hidden_states: Any, router_weight: Any, q: QuantFusedExperts, *, top_k: int,
                                     norm_topk_prob: bool, act_fn: Any, config: dict[str, Any] | None = None,
                                     backend: str = "auto") -> tuple[Any, Any]:
    """W8 grouped version of the sparse-MoE block forward: shared ``_route`` then the kernels."""
    from lemoq.kernels.moe_grouped import _check_act_fn
    from lemoq.kernels.moe_static import _route

    _check_act_fn(act_fn)
    shape = tuple(hidden_states.shape)
    x = hidden_states.reshape(-1, shape[-1])
    logits, top_w, top_i = _route(x, router_weight, top_k=top_k, norm_topk_prob=norm_topk_prob)
    out = grouped_moe_forward_quant(x, q, top_i.reshape(-1), top_w.reshape(-1), config=config, backend=backend)
    return out.reshape(*shape), logits
