"""Per-token symmetric INT8 KV cache: reference maths, guards and the write kernels
(reference: src/lemoq/kernels/kv_int8.py:30-355).

Rounding chain (bit-exact contract): fp32 ``amax`` -> ``scale = amax/127`` (1.0 for a zero row)
-> ``round(x/scale)`` half-to-even with the fp32 scale -> clamp to +-127; the scale is stored
as fp16.
"""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi

_QMAX = 127.0


def quantize_per_token_int8(x: Any) -> tuple[Any, Any]:
    """Per-token symmetric int8 along the last dim of a CUDA fp16 tensor ``(..., D)``:
    returns ``(codes int8 (..., D), scale fp16 (...,))``.  Runs the same CUDA row quantiser as
    the cache write; there is no host implementation."""
    _cabi.require_cuda(x, what="quantize_per_token_int8")
    if x.dtype != torch.float16:
        raise NotImplementedError("quantize_per_token_int8: 只支持 fp16，得到 %s" % x.dtype)
    d = int(x.shape[-1])
    rows = int(x.numel() // max(d, 1))
    xc = x.contiguous()
    codes = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(xc.shape[:-1], dtype=torch.float16, device=x.device)
    if rows == 0:
        return codes, scale
    # the row kernel quantises a K row and a V row per head: feed the same rows to both sides
    spare_c = torch.empty_like(codes)
    spare_s = torch.empty_like(scale)
    _cabi.call("lemoq_kv_int8_cache_write", _cabi.ptr(xc), _cabi.ptr(xc), _cabi.ptr(codes), _cabi.ptr(scale),
               _cabi.ptr(spare_c), _cabi.ptr(spare_s), None, rows, 1, d, None, _cabi.current_stream(x.device))
    return codes, scale


def dequant_int8(codes: Any, scale: Any) -> Any:
    return codes.float() * scale.float()


def fold_scores_per_token_reference(scores: Any, k_scale: Any) -> Any:
    return scores * k_scale


def kv_int8_rows_applicable(k_new: Any, v_new: Any) -> bool:
    """Row guard of the write path: CUDA, fp16, ``(1, H, 1, D)``, contiguous, D a power of two."""
    if not (k_new.is_cuda and v_new.is_cuda):
        return False
    if k_new.dtype is not torch.float16 or v_new.dtype is not torch.float16:
        return False
    if k_new.shape != v_new.shape or k_new.dim() != 4 or k_new.shape[0] != 1 or k_new.shape[2] != 1:
        return False
    if not (k_new.is_contiguous() and v_new.is_contiguous()):
        return False
    dim = int(k_new.shape[-1])
    return dim >= 1 and dim & (dim - 1) == 0


def kv_int8_bulk_quantize(cache_keys: Any, cache_values: Any, filled: Any = None) -> dict[str, Any]:
    """Quantise a whole fp16 cache ``(1, H, S, D)`` into ``kc/ks/vc/vs``.  With ``filled`` in ``[1, S]`` only the
    first ``filled`` slots are quantised and the rest become code 0 / scale 1.  ``filled=None`` quantises every
    slot, and so does ``filled <= 0``: the reference's test is ``filled is not None and filled > 0``
    (src/lemoq/kernels/kv_int8.py:147), so a zero length falls into its whole-cache branch."""
    _, h, s, d = (int(v) for v in cache_keys.shape)
    dev = cache_keys.device
    if filled is not None:
        filled = int(filled.item()) if hasattr(filled, "item") else int(filled)  # the init path may synchronise once
    count = -1 if filled is None or filled <= 0 else min(filled, s)  # -1: every slot
    _cabi.require_cuda(cache_keys, cache_values, what="kv_int8_bulk_quantize")
    if cache_keys.dtype != torch.float16 or cache_values.dtype != torch.float16:
        raise NotImplementedError("kv_int8_bulk_quantize: cache 只支持 fp16")
    keys, values = cache_keys.contiguous(), cache_values.contiguous()
    codes = lambda: torch.empty((1, h, s, d), dtype=torch.int8, device=dev)  # noqa: E731
    scales = lambda: torch.empty((1, h, s), dtype=torch.float16, device=dev)  # noqa: E731
    out = {"kc": codes(), "ks": scales(), "vc": codes(), "vs": scales()}
    _cabi.call("lemoq_kv_int8_bulk_quantize", _cabi.ptr(keys), _cabi.ptr(values), _cabi.ptr(out["kc"]), _cabi.ptr(out["ks"]),
               _cabi.ptr(out["vc"]), _cabi.ptr(out["vs"]), h, s, d, count, _cabi.current_stream(dev))
    return out


def kv_int8_init_buffers(layer_keys: Any, layer_values: Any, filled: Any = None) -> dict[str, Any]:
    bufs = kv_int8_bulk_quantize(layer_keys, layer_values, filled)
    bufs["initialized"] = True
    return bufs


def kv_int8_cache_write(bufs: dict[str, Any], k_new: Any, v_new: Any, pos: Any) -> None:
    """Quantise the new ``(1,H,1,D)`` rows into slot ``pos`` (device int tensor) of the mirror."""
    if not kv_int8_rows_applicable(k_new, v_new):
        raise RuntimeError("kv_int8_cache_write: 行守卫不满足 (row guard failed) - caller must fall back to fp16")
    kc = bufs["kc"]
    if kc.shape[1] != k_new.shape[1] or kc.shape[3] != k_new.shape[3] or kc.shape[0] != 1 or not kc.is_contiguous():
        raise RuntimeError("kv_int8_cache_write: buffer 形状/布局与行不匹配 %s vs %s"
                           % (tuple(kc.shape), tuple(k_new.shape)))
    p = pos.reshape(-1)
    if p.numel() != 1:
        raise ValueError("kv_int8_cache_write: pos must hold one element")
    if p.dtype != torch.int64:
        p = p.to(torch.int64)
    _cabi.call("lemoq_kv_int8_cache_write", _cabi.ptr(k_new), _cabi.ptr(v_new), _cabi.ptr(kc), _cabi.ptr(bufs["ks"]),
               _cabi.ptr(bufs["vc"]), _cabi.ptr(bufs["vs"]), _cabi.ptr(p), int(kc.shape[1]), int(kc.shape[2]),
               int(kc.shape[3]), None, _cabi.current_stream(kc.device))


def kv_int8_write(k_new: Any, v_new: Any, *, k_codes: Any = None, k_scale: Any = None, v_codes: Any = None,
                  v_scale: Any = None) -> tuple[Any, Any, Any, Any]:
    """Quantise ``(1,H,1,D)`` rows into fresh (or given) ``(1,H,1,D)`` int8 + ``(1,H,1)`` fp16 outputs."""
    if not kv_int8_rows_applicable(k_new, v_new):
        raise RuntimeError("kv_int8_write: 守卫不满足 (guard failed) - check kv_int8_rows_applicable first")
    heads, dim = int(k_new.shape[1]), int(k_new.shape[-1])
    if k_codes is None:
        k_codes = torch.empty((1, heads, 1, dim), dtype=torch.int8, device=k_new.device)
        k_scale = torch.empty((1, heads, 1), dtype=torch.float16, device=k_new.device)
        v_codes = torch.empty((1, heads, 1, dim), dtype=torch.int8, device=v_new.device)
        v_scale = torch.empty((1, heads, 1), dtype=torch.float16, device=v_new.device)
    _cabi.call("lemoq_kv_int8_cache_write", _cabi.ptr(k_new), _cabi.ptr(v_new), _cabi.ptr(k_codes), _cabi.ptr(k_scale),
               _cabi.ptr(v_codes), _cabi.ptr(v_scale), None, heads, 1, dim, None, _cabi.current_stream(k_new.device))
    return k_codes, k_scale, v_codes, v_scale
