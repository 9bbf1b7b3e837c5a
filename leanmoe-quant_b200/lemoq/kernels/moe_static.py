"""Fixed-shape (graph-safe) MoE block forward and its installation on a model
(reference: src/lemoq/kernels/moe_static.py).

Dispatch by token count: one token -> the grouped expert kernels (``impl="grouped"``, fp16 or W8
weights) or the fixed-shape gather+bmm form (``impl="gather"``); more than one token (prefill,
eager only) -> the per-expert loop, which reads each expert's weights once.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.nn.functional as F

__all__ = ["FusedExperts", "VALID_MOE_IMPLS", "fuse_experts", "static_moe_forward", "replace_moe_blocks"]

VALID_MOE_IMPLS = ("gather", "grouped")


@dataclass
class FusedExperts:
    """``gate_up (E, 2*ffn, hidden)`` (gate rows first) and ``down (E, hidden, ffn)``."""

    gate_up: Any
    down: Any

    @property
    def num_experts(self) -> int:
        return int(self.gate_up.shape[0])

    def to(self, device: Any = None, dtype: Any = None) -> "FusedExperts":
        if isinstance(device, torch.dtype):
            device, dtype = None, device
        dtype = dtype or self.gate_up.dtype
        device = self.gate_up.device if device is None else device
        return FusedExperts(gate_up=self.gate_up.to(device=device, dtype=dtype).contiguous(),
                            down=self.down.to(device=device, dtype=dtype).contiguous())

    def nbytes(self) -> int:
        return int(self.gate_up.numel() * self.gate_up.element_size()) + int(self.down.numel() * self.down.element_size())


def fuse_experts(experts: Any) -> FusedExperts:
    """Stack a ``ModuleList`` of expert MLPs (``gate_proj/up_proj/down_proj``) into two tensors."""
    layers = list(experts)
    if not layers:
        raise ValueError("experts 是空的 (empty)")
    gate = torch.stack([e.gate_proj.weight.detach() for e in layers], dim=0)
    up = torch.stack([e.up_proj.weight.detach() for e in layers], dim=0)
    down = torch.stack([e.down_proj.weight.detach() for e in layers], dim=0)
    return FusedExperts(gate_up=torch.cat([gate, up], dim=1).contiguous(), down=down.contiguous())


def _is_quant_fused(fused: Any) -> bool:
    from lemoq.kernels.moe_grouped_quant import QuantFusedExperts

    return isinstance(fused, QuantFusedExperts)


def _fused_route_enabled() -> bool:
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("fused_route")


def _route(x: Any, router_weight: Any, *, top_k: int, norm_topk_prob: bool):
    """Router: ``(logits (T,E), top_w (T,K) x.dtype, top_i (T,K) int64)``.  The linear layer is
    ``F.linear``; softmax + top-k run in one CUDA kernel when ``fused_route`` is on and the logits
    are on the GPU, else through ATen (bit-identical selection when there is no tie)."""
    logits = F.linear(x, router_weight)
    if _fused_route_enabled() and logits.is_cuda:
        from lemoq.kernels.routing import routing_softmax_topk

        top_w, top_i = routing_softmax_topk(logits, top_k=top_k, norm_topk_prob=norm_topk_prob)
        return logits, top_w.to(x.dtype), top_i
    weights = F.softmax(logits, dim=-1, dtype=torch.float)
    top_w, top_i = torch.topk(weights, top_k, dim=-1)
    if norm_topk_prob:
        top_w = top_w / top_w.sum(dim=-1, keepdim=True)
    return logits, top_w.to(x.dtype), top_i


def static_moe_forward(hidden_states: Any, router_weight: Any, fused: Any, *, top_k: int, norm_topk_prob: bool = False,
                       act_fn: Callable[[Any], Any] | None = None, impl: str = "gather",
                       moe_config: dict[str, Any] | None = None) -> tuple[Any, Any]:
    """MoE block forward, returns ``(output, router_logits)``.  ``impl`` only affects the
    one-token decode; prefill always takes the per-expert loop."""
    if impl not in VALID_MOE_IMPLS:
        raise ValueError("unknown impl %r; expected one of %s" % (impl, VALID_MOE_IMPLS))
    act_fn = F.silu if act_fn is None else act_fn
    shape = tuple(hidden_states.shape)
    hidden = shape[-1]
    tokens = 1
    for s in shape[:-1]:
        tokens *= s
    x = hidden_states.reshape(tokens, hidden)
    if tokens == 1:
        if impl == "grouped":
            if _is_quant_fused(fused):
                from lemoq.kernels.moe_grouped_quant import static_moe_forward_grouped_quant

                return static_moe_forward_grouped_quant(hidden_states, router_weight, fused, top_k=top_k,
                                                        norm_topk_prob=norm_topk_prob, act_fn=act_fn, config=moe_config)
            from lemoq.kernels.moe_grouped import static_moe_forward_grouped

            return static_moe_forward_grouped(hidden_states, router_weight, fused, top_k=top_k,
                                              norm_topk_prob=norm_topk_prob, act_fn=act_fn, config=moe_config)
        return _decode_forward(x, router_weight, fused, top_k=top_k, norm_topk_prob=norm_topk_prob, act_fn=act_fn,
                               out_shape=shape, hidden=hidden)
    out, logits = _prefill_forward(x, router_weight, fused, top_k=top_k, norm_topk_prob=norm_topk_prob, act_fn=act_fn)
    return out.reshape(*shape), logits


def _decode_forward(x: Any, router_weight: Any, fused: FusedExperts, *, top_k: int, norm_topk_prob: bool,
                    act_fn: Callable[[Any], Any], out_shape: tuple, hidden: int) -> tuple[Any, Any]:
    """Fixed-shape gather + bmm (tensor indexing only; no data-dependent shape)."""
    logits, top_w, top_i = _route(x, router_weight, top_k=top_k, norm_topk_prob=norm_topk_prob)
    tokens = int(x.shape[0])
    ids = top_i.reshape(-1)
    xr = x.repeat_interleave(top_k, dim=0)
    gu = torch.bmm(fused.gate_up[ids], xr.unsqueeze(-1)).squeeze(-1)
    gate, up = gu.chunk(2, dim=-1)
    act = act_fn(gate) * up
    y = torch.bmm(fused.down[ids], act.unsqueeze(-1)).squeeze(-1) * top_w.reshape(-1, 1)
    return y.reshape(tokens, top_k, hidden).sum(dim=1).reshape(*out_shape), logits


def _prefill_forward(x: Any, router_weight: Any, fused: Any, *, top_k: int, norm_topk_prob: bool,
                     act_fn: Callable[[Any], Any]) -> tuple[Any, Any]:
    """Prefill only (eager; data-dependent ``nonzero``, never captured): every expert's weights
    are read once and applied to all tokens routed to it.  W8 experts are dequantised one at a time."""
    logits, top_w, top_i = _route(x, router_weight, top_k=top_k, norm_topk_prob=norm_topk_prob)
    out = torch.zeros_like(x)
    quant = _is_quant_fused(fused)
    for e in range(fused.num_experts):
        tok, slot = (top_i == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        w = top_w[tok, slot].unsqueeze(-1)
        xe = x[tok]
        if quant:
            gu_w = fused.dequant_gate_up_expert(e, dtype=x.dtype)
            dn_w = fused.dequant_down_expert(e, dtype=x.dtype)
        else:
            gu_w, dn_w = fused.gate_up[e], fused.down[e]
        gate, up = (xe @ gu_w.t()).chunk(2, dim=-1)
        y = (act_fn(gate) * up) @ dn_w.t()
        out.index_add_(0, tok, y * w)
    return out, logits


class StaticShapedMoE:
    """Holds the fused (optionally W8-quantised) experts and the router of one MoE block."""

    def __init__(self, block: Any, *, device: Any = None, dtype: Any = None, impl: str = "gather", quant: Any = None) -> None:
        if impl not in VALID_MOE_IMPLS:
            raise ValueError("unknown impl %r; expected one of %s" % (impl, VALID_MOE_IMPLS))
        bits = getattr(quant, "weight_bits", None) if quant is not None else None
        if bits is not None and impl != "grouped":
            raise NotImplementedError("量化 × %s 的路径不存在：量化只接在 grouped 的 fused 张量上" % impl)
        self.impl = impl
        self.top_k = int(block.top_k)
        self.norm_topk_prob = bool(getattr(block, "norm_topk_prob", False))
        self.act_fn = getattr(block, "act_fn", None)
        self.router_weight = block.gate.weight.detach()
        fused = fuse_experts(block.experts)
        if bits is None:
            self.fused = fused if device is None and dtype is None else fused.to(device or fused.gate_up.device, dtype=dtype)
        else:
            from lemoq.kernels.moe_grouped_quant import quantize_fused_experts

            self.fused = quantize_fused_experts(fused, bits=int(bits), group_size=int(getattr(quant, "group_size", 128) or 128))
            del fused

    def __call__(self, hidden_states: Any) -> tuple[Any, Any]:
        return static_moe_forward(hidden_states, self.router_weight, self.fused, top_k=self.top_k,
                                  norm_topk_prob=self.norm_topk_prob, act_fn=self.act_fn, impl=self.impl)


def replace_moe_blocks(model: Any, *, verbose: bool = False, impl: str = "gather", quant: Any = None,
                       prequantized: dict[int, Any] | None = None) -> int:
    """Replace every sparse-MoE block's forward in place; the original expert modules are freed.
    ``quant`` (a ``SchemeSpec`` with 8 weight bits) quantises the fused tensors on the spot;
    ``prequantized`` maps layer index -> ``QuantFusedExperts`` and skips quantisation.  Must run
    before capture."""
    if impl not in VALID_MOE_IMPLS:
        raise ValueError("unknown impl %r; expected one of %s" % (impl, VALID_MOE_IMPLS))
    if prequantized is not None:
        if impl != "grouped" or quant is not None:
            raise ValueError("prequantized requires grouped and forbids re-quantization")
        if set(prequantized) != set(range(len(model.model.layers))):
            raise ValueError("prequantized must cover all model layers exactly")
    replaced = 0
    for index, layer in enumerate(model.model.layers):
        block = getattr(layer, "mlp", None)
        if block is None or not hasattr(block, "experts") or not hasattr(block, "gate") or not hasattr(block, "top_k"):
            continue
        if prequantized is None:
            static = StaticShapedMoE(block, impl=impl, quant=quant)
            fused, router = static.fused, static.router_weight
        else:
            fused, router = prequantized[index].to(device=block.gate.weight.device), block.gate.weight.detach()
        del block.experts
        block._static_experts = fused
        block._static_router = router
        block._static_top_k = int(block.top_k)
        block._static_norm = bool(getattr(block, "norm_topk_prob", False))
        block._static_act = getattr(block, "act_fn", None)
        block._static_impl = impl

        def _forward(hidden_states, _b=block):
            return static_moe_forward(hidden_states, _b._static_router, _b._static_experts, top_k=_b._static_top_k,
                                      norm_topk_prob=_b._static_norm, act_fn=_b._static_act, impl=_b._static_impl)

        block.forward = _forward
        replaced += 1
        if verbose:
            print("  replaced MoE block %d" % replaced)
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return replaced
