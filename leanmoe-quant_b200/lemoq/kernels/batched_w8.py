"""W8 linears and grouped experts for MANY tokens per call (batched decode): weights-stationary kernels on the int8
tensor-core tile, every weight byte read once per block of tokens.  The reference's T > 1 arms dequantise and call a dense matmul
(`quant/linear.py:365`, `moe_static.py:329`); these compute the same sums with exact integer partial sums.
CUDA only: there is no CPU path."""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi


def quantise_tokens(x: Any) -> Any:
    """``x (T, K)`` fp16 contiguous -> opaque digit-plane buffer for :func:`w8_rows_tokens`."""
    if x.dim() != 2 or x.dtype != torch.float16 or not x.is_contiguous():
        raise ValueError("x 必须是连续的 (T, K) fp16")
    _cabi.require_cuda(x, what="batched W8 kernels")
    t, k = int(x.shape[0]), int(x.shape[1])
    planes = torch.empty(max(int(_cabi.lib().lemoq_w8_token_planes_bytes(max(t, 1), k)), 16), dtype=torch.uint8, device=x.device)
    _cabi.call("lemoq_w8_quantise_tokens", _cabi.ptr(x), t, k, _cabi.ptr(planes), _cabi.current_stream(x.device))
    return planes


def w8_rows_tokens(planes: Any, tokens: int, codes: Any, scale: Any, *, group_size: int, seg_offsets: Any = None,
                   gate_up: bool = False) -> Any:
    """``codes (N, K)`` or ``(E, N, K)`` int8, ``scale`` matching fp16 -> ``(T, N)`` fp16, or ``(T, N/2)`` =
    silu(gate) * up when ``gate_up``.  ``seg_offsets (E+1,)`` int32: tokens ``[seg[e], seg[e+1])`` use expert e."""
    if codes.dtype != torch.int8 or scale.dtype != torch.float16:
        raise ValueError("codes 必须 int8，scale 必须 fp16")
    if not (codes.is_contiguous() and scale.is_contiguous()):
        raise ValueError("codes/scale 必须连续")
    e = int(codes.shape[0]) if codes.dim() == 3 else 1
    n, k = int(codes.shape[-2]), int(codes.shape[-1])
    if e > 1 and (seg_offsets is None or seg_offsets.dtype != torch.int32 or int(seg_offsets.numel()) != e + 1):
        raise ValueError("多专家调用需要 (E+1,) int32 的 seg_offsets")
    out = torch.empty((tokens, n // 2 if gate_up else n), dtype=torch.float16, device=codes.device)
    _cabi.call("lemoq_w8_rows_tokens", _cabi.ptr(planes), tokens, _cabi.ptr(codes), _cabi.ptr(scale), n, k, int(group_size),
               _cabi.ptr(seg_offsets) if seg_offsets is not None else None, e, 1 if gate_up else 0, _cabi.ptr(out),
               _cabi.current_stream(codes.device))
    return out


def w8_linear_tokens(x: Any, codes: Any, scale: Any, *, group_size: int) -> Any:
    """``x (T, K)`` fp16 -> ``(T, N)`` fp16 through a W8 linear ``codes (N, K)``."""
    return w8_rows_tokens(quantise_tokens(x.contiguous()), int(x.shape[0]), codes, scale, group_size=group_size)


def expert_segments(expert_ids: Any, experts: int) -> Any:
    """``(experts + 1,)`` int32 offsets of the segments of ``expert_ids`` (ascending local ids): rows ``[seg[e], seg[e+1])``
    belong to expert e.  No data-dependent shape and no host read: usable under stream capture.  Ids ``>= experts``
    (padding rows of a static-capacity exchange, sorted behind the real ones) belong to no segment."""
    counts = (expert_ids.reshape(-1, 1) == torch.arange(experts, device=expert_ids.device).reshape(1, -1)).sum(dim=0)
    seg = torch.zeros(experts + 1, dtype=torch.int32, device=expert_ids.device)
    seg[1:] = torch.cumsum(counts, dim=0).to(torch.int32)
    return seg


def w8_experts_tokens(x: Any, expert_ids: Any, gate_up: Any, gate_up_scale: Any, down: Any, down_scale: Any, *,
                      group_size: int, seg_offsets: Any = None) -> Any:
    """Grouped experts on rows SORTED by expert: ``x (R, H)`` fp16, ``expert_ids (R,)`` ascending local ids ->
    ``(R, H)`` fp16 unweighted expert outputs (gate/up + SwiGLU, then down).  Rows whose id is >= the number of
    experts must come last; their outputs are left unwritten.  ``seg_offsets`` (from :func:`expert_segments`) may be
    handed in by a caller that already has it."""
    rows = int(x.shape[0])
    seg = expert_segments(expert_ids, int(gate_up.shape[0])) if seg_offsets is None else seg_offsets
    act = w8_rows_tokens(quantise_tokens(x.contiguous()), rows, gate_up, gate_up_scale, group_size=group_size, seg_offsets=seg, gate_up=True)
    return w8_rows_tokens(quantise_tokens(act), rows, down, down_scale, group_size=group_size, seg_offsets=seg)
