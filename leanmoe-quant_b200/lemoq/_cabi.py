"""ctypes binding of ``liblemoq_b200.so`` (the C-ABI declared in ``include/lemoq_b200.h``).

The library is the only implementation of the decode kernels: there is no CPU or
eager fallback.  ``lib()`` raises ``RuntimeError`` when the shared object is missing,
and every kernel wrapper in :mod:`lemoq.kernels` goes through ``call()``, which maps
the C status codes onto the exception types the reference raises
(``ValueError`` / ``NotImplementedError`` / ``RuntimeError``).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from typing import Any

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "csrc", "liblemoq_b200.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA = 0, 1, 2, 3
DTYPE_F16, DTYPE_F32 = 0, 1
FLAG_BAD_POSITION, FLAG_BAD_LENGTH, FLAG_BAD_EXPERT = 1, 2, 4

_lib = None
_load_error: str | None = None


class LayerDesc(Structure):
    _fields_ = [(n, c_void_p) for n in (
        "ln1", "ln2", "q_norm", "k_norm", "qkv_codes", "qkv_scale", "o_codes", "o_scale", "router",
        "gu_codes", "gu_scale", "dn_codes", "dn_scale", "keys", "values", "kc", "ks", "vc", "vs")]


class StepDesc(Structure):
    _fields_ = (
        [(n, c_int) for n in ("layers", "hidden", "heads", "head_dim", "experts", "top_k", "ffn", "vocab",
                              "group_size", "max_len")]
        + [("eps", c_float)]
        + [(n, c_int) for n in ("norm_topk_prob", "kv_int8", "attn_splits", "use_pdl")]
        + [(n, c_void_p) for n in ("embed", "final_norm", "lm_head_codes", "lm_head_scale", "rope_cos", "rope_sin",
                                   "token", "cache_position", "filled_len", "logits", "workspace")]
        + [("workspace_bytes", c_size_t), ("next_token", c_void_p), ("self_feed", c_int), ("token_log", c_void_p)]
    )


_SIGNATURES = {
    "lemoq_version": (c_char_p, []),
    "lemoq_last_error": (c_char_p, []),
    "lemoq_set_tuning": (c_int, [c_int, c_int]),
    "lemoq_rtn_quantize_w8": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "lemoq_dequant_gemv_w8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "lemoq_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p]),
    "lemoq_rope_qk": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p,
                              c_void_p, c_void_p]),
    "lemoq_kv_direct_write": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_void_p, c_void_p]),
    "lemoq_kv_int8_cache_write": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                          c_int, c_int, c_void_p, c_void_p]),
    "lemoq_kv_int8_bulk_quantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_int, c_void_p]),
    "lemoq_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "lemoq_attn_decode_fp16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
                                       c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "lemoq_attn_decode_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "lemoq_w8_token_planes_bytes": (c_size_t, [c_int, c_int]),
    "lemoq_w8_quantise_tokens": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "lemoq_w8_rows_tokens": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                     c_void_p, c_void_p]),
    "lemoq_ep_dispatch": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p]),
    "lemoq_ep_regroup": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lemoq_ep_return": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "lemoq_ep_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "lemoq_attn_static_scratch_bytes": (c_size_t, []),
    "lemoq_attn_decode_int8_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                              c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "lemoq_routing_softmax_topk": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                           c_void_p]),
    "lemoq_route": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p]),
    "lemoq_moe_grouped_w8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lemoq_moe_gate_up_w8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p]),
    "lemoq_moe_down_w8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_void_p, c_void_p]),
    "lemoq_moe_grouped_fp16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lemoq_step_workspace_bytes": (c_size_t, [POINTER(StepDesc)]),
    "lemoq_step_create": (c_int, [POINTER(StepDesc), POINTER(LayerDesc), POINTER(c_void_p)]),
    "lemoq_step_destroy": (None, [c_void_p]),
    "lemoq_step_run": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
    "lemoq_step_error_flag": (c_void_p, [c_void_p]),
    "lemoq_step_topk_ids": (c_void_p, [c_void_p]),
    "lemoq_step_router_logits": (c_void_p, [c_void_p]),
    "lemoq_step_phase_stamps": (c_void_p, [c_void_p]),
    "lemoq_step_engine": (ctypes.c_char_p, [c_void_p]),
}

EXPORTED_SYMBOLS = tuple(sorted(_SIGNATURES))


def available() -> bool:
    """True when the shared library can be loaded (does not need a GPU)."""
    try:
        lib()
    except RuntimeError:
        return False
    return True


def unavailable_reason() -> str | None:
    if available():
        return None
    return _load_error


def lib() -> Any:
    """The loaded library.  Fails loudly when it has not been built."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        _load_error = (
            "lemoq CUDA library not built: %s is missing (run `python leanmoe-quant_b200/csrc/build.py`); "
            "there is no CPU fallback" % LIB_PATH
        )
        raise RuntimeError(_load_error)
    try:
        handle = ctypes.CDLL(LIB_PATH)
    except OSError as exc:
        _load_error = "cannot load lemoq CUDA library %s: %s" % (LIB_PATH, exc)
        raise RuntimeError(_load_error) from exc
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


def last_error() -> str:
    return (lib().lemoq_last_error() or b"").decode("utf-8", "replace")


def check(status: int, what: str = "") -> None:
    if status == OK:
        return
    msg = "%s%s" % (what + ": " if what else "", last_error())
    if status == ERR_INVALID:
        raise ValueError(msg)
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError("CUDA kernel path failed: " + msg)


def call(name: str, *args: Any) -> None:
    check(getattr(lib(), name)(*args), name)


def ptr(t: Any) -> int | None:
    """Device (or host) address of a tensor, ``None`` for ``None``."""
    return None if t is None else int(t.data_ptr())


def current_stream(device: Any = None) -> int:
    import torch

    return int(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors: Any, what: str = "lemoq kernel") -> None:
    """The kernels only exist for CUDA tensors; anything else is an error, not a fallback."""
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("%s 需要 CUDA 张量 (needs CUDA tensors); there is no CPU path" % what)
