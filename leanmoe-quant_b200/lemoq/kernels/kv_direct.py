"""KV direct write (reference: src/lemoq/kernels/kv_direct.py:38-137): bit copy of the RoPE'd K row
and the V row into slot ``cache_position`` of the static fp16 cache, position read on the device."""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi


def kv_direct_write_applicable(cache_layer: Any, key_states: Any, value_states: Any) -> bool:
    """Shape/layout guard; ``False`` means the caller takes the cache's own ``update()``."""
    if not (key_states.is_cuda and value_states.is_cuda):
        return False
    keys = getattr(cache_layer, "keys", None)
    values = getattr(cache_layer, "values", None)
    if keys is None or values is None or not (keys.is_cuda and values.is_cuda):
        return False
    if keys.shape != values.shape or keys.dim() != 4 or keys.shape[0] != 1:
        return False
    if not (keys.is_contiguous() and values.is_contiguous()):
        return False
    if key_states.dtype is not keys.dtype or value_states.dtype is not values.dtype:
        return False
    if keys.dtype is not torch.float16:
        return False
    _, heads, _, dim = keys.shape
    if key_states.shape != (1, heads, 1, dim) or value_states.shape != (1, heads, 1, dim):
        return False
    if key_states.stride(3) != 1 or value_states.stride(3) != 1 or key_states.stride(1) != value_states.stride(1):
        return False
    return dim >= 2 and (dim & (dim - 1)) == 0


def kv_direct_write(layer: Any, key_states: Any, value_states: Any, cache_position: Any) -> None:
    """Write the ``(1,H,1,D)`` rows into ``layer.keys/values[:, :, pos]``.  ``cache_position`` is a
    one-element int64 device tensor."""
    if not torch.cuda.is_available():
        raise RuntimeError("kv_direct_write 需要 CUDA")
    pos = cache_position.reshape(-1)
    if pos.numel() != 1:
        raise ValueError("kv_direct_write 只支持 decode 的单槽写（q_len=1）")
    if pos.dtype != torch.int64:
        pos = pos.to(torch.int64)
    _, heads, max_len, dim = layer.keys.shape
    _cabi.call("lemoq_kv_direct_write", _cabi.ptr(key_states), _cabi.ptr(value_states), int(key_states.stride(1)),
               _cabi.ptr(layer.keys), _cabi.ptr(layer.values), _cabi.ptr(pos), int(heads), int(max_len), int(dim),
               None, _cabi.current_stream(layer.keys.device))
