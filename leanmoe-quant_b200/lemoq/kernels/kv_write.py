"""Semantic contract of the KV slot write (reference: src/lemoq/kernels/kv_write.py:28-50)."""

from __future__ import annotations

from typing import Any


def write_kv_slot(cache: Any, layer_idx: int, pos: int, key_states: Any, value_states: Any) -> tuple[Any, Any]:
    """Write ``(b, h, q_len, d)`` new K/V into ``cache.layers[layer_idx]`` at ``[pos, pos+q_len)`` in
    place (same buffers, no other slot touched).  Device independent; the CUDA kernel of
    :mod:`lemoq.kernels.kv_direct` must produce the same bits."""
    layer = cache.layers[layer_idx]
    if not layer.is_initialized:
        layer.lazy_initialization(key_states)
    q_len = key_states.shape[2]
    layer.keys[:, :, pos: pos + q_len, :] = key_states
    layer.values[:, :, pos: pos + q_len, :] = value_states
    return layer.keys, layer.values
