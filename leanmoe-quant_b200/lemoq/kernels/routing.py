"""Router softmax + top-k on the GPU (reference: src/lemoq/kernels/_routing_triton.py:88-130)."""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi

__all__ = ["routing_softmax_topk"]


def routing_softmax_topk(logits: Any, *, top_k: int, norm_topk_prob: bool = False) -> tuple[Any, Any]:
    """``(T, E)`` logits -> ``(top_w fp32 (T, K), top_i int64 (T, K))``.

    fp32 softmax, K rounds of arg-max with the lowest index winning ties, optional
    renormalisation by the selected weights' sum.  The router linear layer is not part
    of this op.  CUDA tensors only; a CPU tensor raises ``RuntimeError``.
    """
    if not torch.is_tensor(logits):
        raise TypeError("logits 必须为张量 (must be a tensor)")
    if logits.ndim != 2:
        raise ValueError("logits 必须是 (T, E)，得到 shape %s" % (tuple(logits.shape),))
    t, e = int(logits.shape[0]), int(logits.shape[1])
    if type(top_k) is not int or not (0 < top_k <= e):
        raise ValueError("top_k=%r 必须是 (0, %d] 内的整数" % (top_k, e))
    if not logits.is_floating_point():
        raise ValueError("logits 必须为浮点张量 (must be floating point)")
    top_w = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
    top_i = torch.empty((t, top_k), dtype=torch.int64, device=logits.device)
    if t == 0:
        return top_w, top_i
    if not torch.cuda.is_available():
        raise RuntimeError("routing_softmax_topk 需要 CUDA (needs CUDA)")
    if not logits.is_cuda:
        raise RuntimeError("routing_softmax_topk 需要 CUDA 张量 (needs a CUDA tensor)")
    x = logits
    if x.dtype not in (torch.float16, torch.float32):
        x = x.float()
    if x.stride(1) != 1:
        x = x.contiguous()
    dt = _cabi.DTYPE_F16 if x.dtype == torch.float16 else _cabi.DTYPE_F32
    _cabi.call("lemoq_routing_softmax_topk", _cabi.ptr(x), dt, int(x.stride(0)), t, e, top_k,
               int(bool(norm_topk_prob)), _cabi.ptr(top_w), _cabi.ptr(top_i), _cabi.current_stream(x.device))
    return top_w, top_i
