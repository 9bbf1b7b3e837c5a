"""Sparse-MoE block forward with shapes that never depend on the routing result, and its installation on a model
(the interface of the reference's src/lemoq/kernels/moe_static.py: ``FusedExperts`` :56, ``static_moe_forward`` :170,
``replace_moe_blocks`` :440).

Which code serves a call depends on the token count alone.  One token (decode, capturable): ``impl="grouped"`` runs the
two grouped expert kernels on fp16 or W8 stacks, ``impl="gather"`` a gather + two batched matrix products.  More than
one token (prefill, eager only): a loop over experts in which each expert's weights are read once for all of its
tokens.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.nn.functional as F

__all__ = ["FusedExperts", "VALID_MOE_IMPLS", "fuse_experts", "static_moe_forward", "replace_moe_blocks"]

VALID_MOE_IMPLS = ("gather", "grouped")
_BLOCK_PARTS = ("experts", "gate", "top_k")


def _known_impl(impl: str) -> str:
    if impl not in VALID_MOE_IMPLS:
        raise ValueError("unknown impl %r; expected one of %s" % (impl, VALID_MOE_IMPLS))
    return impl


def _bytes(t: Any) -> int:
    return int(t.numel() * t.element_size())


@dataclass
class FusedExperts:
    """All experts of one block as two stacks: ``gate_up (E, 2*ffn, hidden)`` with the gate rows first, and
    ``down (E, hidden, ffn)``."""

    gate_up: Any
    down: Any

    @property
    def num_experts(self) -> int:
        return int(self.gate_up.shape[0])

    def to(self, device: Any = None, dtype: Any = None) -> "FusedExperts":
        """``.to(device)``, ``.to(dtype)`` or both; the result is contiguous."""
        if isinstance(device, torch.dtype):
            device, dtype = None, device
        move = lambda t: t.to(device=t.device if device is None else device, dtype=dtype or t.dtype).contiguous()  # noqa: E731
        return FusedExperts(gate_up=move(self.gate_up), down=move(self.down))

    def nbytes(self) -> int:
        return _bytes(self.gate_up) + _bytes(self.down)


def fuse_experts(experts: Any) -> FusedExperts:
    """Stack a list of expert MLPs (``gate_proj`` / ``up_proj`` / ``down_proj``) into a :class:`FusedExperts`."""
    members = list(experts)
    if not members:
        raise ValueError("experts 是空的 (empty)")
    stack = lambda role: torch.stack([getattr(e, role).weight.detach() for e in members])  # noqa: E731
    return FusedExperts(gate_up=torch.cat((stack("gate_proj"), stack("up_proj")), dim=1).contiguous(),
                        down=stack("down_proj").contiguous())


def _is_quant_fused(fused: Any) -> bool:
    from lemoq.kernels.moe_grouped_quant import QuantFusedExperts

    return isinstance(fused, QuantFusedExperts)


def _fused_route_enabled() -> bool:
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("fused_route")


def _route(x: Any, router_weight: Any, *, top_k: int, norm_topk_prob: bool):
    """``(logits (T,E), top_w (T,K) in x.dtype, top_i (T,K) int64)``.  The logits are a plain ``F.linear``.  Softmax
    and top-k are ONE CUDA kernel when the ``fused_route`` switch is on and the logits live on the GPU, and ATen
    otherwise; without ties both select the same experts."""
    logits = F.linear(x, router_weight)
    if logits.is_cuda and _fused_route_enabled():
        from lemoq.kernels.routing import routing_softmax_topk

        top_w, top_i = routing_softmax_topk(logits, top_k=top_k, norm_topk_prob=norm_topk_prob)
    else:
        top_w, top_i = F.softmax(logits, dim=-1, dtype=torch.float).topk(top_k, dim=-1)
        if norm_topk_prob:
            top_w = top_w / top_w.sum(dim=-1, keepdim=True)
    return logits, top_w.to(x.dtype), top_i


def _one_token_gather(x: Any, router_weight: Any, fused: FusedExperts, *, top_k: int, norm_topk_prob: bool,
                      act_fn: Callable[[Any], Any]) -> tuple[Any, Any]:
    """``impl="gather"``: index the stacks with the chosen expert ids and run two batched matrix-vector products.
    Indexing with a tensor keeps every shape fixed, so the call can be captured."""
    logits, top_w, top_i = _route(x, router_weight, top_k=top_k, norm_topk_prob=norm_topk_prob)
    chosen = top_i.reshape(-1)                                     # (T*K,)
    column = x.repeat_interleave(top_k, dim=0).unsqueeze(-1)       # (T*K, hidden, 1)
    gate, up = torch.bmm(fused.gate_up[chosen], column).squeeze(-1).chunk(2, dim=-1)
    per_expert = torch.bmm(fused.down[chosen], (act_fn(gate) * up).unsqueeze(-1)).squeeze(-1)
    weighted = per_expert * top_w.reshape(-1, 1)
    return weighted.view(x.shape[0], top_k, x.shape[1]).sum(dim=1), logits


def _many_tokens(x: Any, router_weight: Any, fused: Any, *, top_k: int, norm_topk_prob: bool,
                 act_fn: Callable[[Any], Any]) -> tuple[Any, Any]:
    """Prefill (eager: the token lists have data-dependent lengths).  Per expert that received tokens: its weights,
    dequantised on the spot for a W8 stack, applied to those tokens and added into the output rows."""
    logits, top_w, top_i = _route(x, router_weight, top_k=top_k, norm_topk_prob=norm_topk_prob)
    if _is_quant_fused(fused):
        weights_of = lambda e: (fused.dequant_gate_up_expert(e, dtype=x.dtype), fused.dequant_down_expert(e, dtype=x.dtype))  # noqa: E731
    else:
        weights_of = lambda e: (fused.gate_up[e], fused.down[e])  # noqa: E731
    out = torch.zeros_like(x)
    for expert in range(fused.num_experts):
        rows, slots = torch.nonzero(top_i == expert, as_tuple=True)
        if rows.numel():
            gate_up, down = weights_of(expert)
            gate, up = F.linear(x[rows], gate_up).chunk(2, dim=-1)
            out.index_add_(0, rows, F.linear(act_fn(gate) * up, down) * top_w[rows, slots].unsqueeze(-1))
    return out, logits


def static_moe_forward(hidden_states: Any, router_weight: Any, fused: Any, *, top_k: int, norm_topk_prob: bool = False,
                       act_fn: Callable[[Any], Any] | None = None, impl: str = "gather",
                       moe_config: dict[str, Any] | None = None) -> tuple[Any, Any]:
    """Forward of one sparse-MoE block: ``(output shaped like the input, router logits (tokens, experts))``.
    ``impl`` chooses the one-token path only."""
    _known_impl(impl)
    common = dict(top_k=top_k, norm_topk_prob=norm_topk_prob, act_fn=act_fn or F.silu)
    rows = hidden_states.reshape(-1, hidden_states.shape[-1])
    if rows.shape[0] != 1:
        out, logits = _many_tokens(rows, router_weight, fused, **common)
    elif impl == "gather":
        out, logits = _one_token_gather(rows, router_weight, fused, **common)
    else:
        if _is_quant_fused(fused):
            from lemoq.kernels.moe_grouped_quant import static_moe_forward_grouped_quant as grouped
        else:
            from lemoq.kernels.moe_grouped import static_moe_forward_grouped as grouped
        return grouped(hidden_states, router_weight, fused, config=moe_config, **common)
    return out.reshape(hidden_states.shape), logits


class StaticShapedMoE:
    """The router and the fused (optionally W8) experts of one block, callable like the block."""

    def __init__(self, block: Any, *, device: Any = None, dtype: Any = None, impl: str = "gather", quant: Any = None) -> None:
        self.impl = _known_impl(impl)
        bits = getattr(quant, "weight_bits", None)
        if bits is not None and impl != "grouped":
            raise NotImplementedError("量化 × %s 的路径不存在: quantised experts exist for impl='grouped' only" % impl)
        self.top_k, self.norm_topk_prob = int(block.top_k), bool(getattr(block, "norm_topk_prob", False))
        self.act_fn = getattr(block, "act_fn", None)
        self.router_weight = block.gate.weight.detach()
        stacks = fuse_experts(block.experts)
        if bits is not None:
            from lemoq.kernels.moe_grouped_quant import quantize_fused_experts

            stacks = quantize_fused_experts(stacks, bits=int(bits), group_size=int(getattr(quant, "group_size", None) or 128))
        elif device is not None or dtype is not None:
            stacks = stacks.to(device, dtype=dtype)
        self.fused = stacks

    def __call__(self, hidden_states: Any) -> tuple[Any, Any]:
        return static_moe_forward(hidden_states, self.router_weight, self.fused, top_k=self.top_k,
                                  norm_topk_prob=self.norm_topk_prob, act_fn=self.act_fn, impl=self.impl)


def _block_forward(block: Any) -> Callable[[Any], tuple[Any, Any]]:
    def forward(hidden_states: Any) -> tuple[Any, Any]:
        return static_moe_forward(hidden_states, block._static_router, block._static_experts, top_k=block._static_top_k,
                                  norm_topk_prob=block._static_norm, act_fn=block._static_act, impl=block._static_impl)

    return forward


def replace_moe_blocks(model: Any, *, verbose: bool = False, impl: str = "gather", quant: Any = None,
                       prequantized: dict[int, Any] | None = None) -> int:
    """Give every sparse-MoE block of ``model`` the fixed-shape forward and free its expert modules; returns the
    number of blocks.  ``quant`` (a spec with 8 weight bits) quantises the stacks as they are built; ``prequantized``
    (layer index -> ``QuantFusedExperts``, one per layer) supplies finished stacks instead.  Call before capture."""
    _known_impl(impl)
    decoder_layers = model.model.layers
    if prequantized is not None:
        if impl != "grouped" or quant is not None:
            raise ValueError("prequantized requires grouped and forbids re-quantization")
        if sorted(prequantized) != list(range(len(decoder_layers))):
            raise ValueError("prequantized must cover all model layers exactly")
        # every payload is checked before the first block is touched: a bad one leaves the model as it was
        from lemoq.quant.expert_calibration import validate_packed

        for index, layer in enumerate(decoder_layers):
            members = getattr(getattr(layer, "mlp", None), "experts", None)
            if members is not None:
                validate_packed(prequantized[index], experts=len(members), hidden=int(members[0].gate_proj.in_features),
                                ffn=int(members[0].down_proj.in_features))
    count = 0
    for index, layer in enumerate(decoder_layers):
        block = getattr(layer, "mlp", None)
        if block is None or not all(hasattr(block, part) for part in _BLOCK_PARTS):
            continue  # a dense layer
        router = block.gate.weight.detach()
        if prequantized is not None:
            stacks = prequantized[index].to(device=router.device)
        else:
            stacks = StaticShapedMoE(block, impl=impl, quant=quant).fused
        del block.experts
        block._static_experts, block._static_router, block._static_impl = stacks, router, impl
        block._static_top_k = int(block.top_k)
        block._static_norm = bool(getattr(block, "norm_topk_prob", False))
        block._static_act = getattr(block, "act_fn", None)
        block.forward = _block_forward(block)
        count += 1
        if verbose:
            print("  replaced MoE block %d" % count)
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return count
