"""Split-KV decode attention for batch 1, one query row: the operator surface of the reference's
src/lemoq/kernels/attn_decode.py (``attn_decode_forward`` :509, ``attn_decode_forward_int8`` :620, ``launch_plan``
:237, ``replace_attention_cores`` :1027) over ONE CUDA launch.

The launch computes a partial (max, sum, weighted values) per split of the key range and the last block of each head
merges the splits in a fixed order, so results do not depend on scheduling.  The filled length is a device scalar the
kernel reads: the launch shape is static and a captured graph serves every step.  Keys and values are either the fp16
cache itself or its int8 mirror with one fp16 scale per (head, position); the scales are folded into the scores and
the softmax weights.

Layout of this file: constants and gates, the operand records (every shape/dtype/stride rule of a call is one line
of a rule list), the two operators, and the wiring into OLMoE attention modules.
"""

from __future__ import annotations

import copy
import math
import types
import weakref
from dataclasses import dataclass
from typing import Any, Callable, Iterable

import torch

from lemoq import _cabi

__all__ = [
    "PARITY_GATE", "LENGTH_CHANGE_GATE", "ATTN_CONFIGS", "LOG2E", "attn_decode_available", "merged_config",
    "resolve_num_splits", "launch_plan", "attn_decode_forward", "attn_decode_forward_int8", "judge_length_change",
    "warm", "replace_attention_cores", "restore_attention_cores", "attention_cores_replaced", "decode_call_count",
    "attention_int8_runs",
]

LOG2E = 1.4426950408889634

# Both gates were fixed before anything was measured; the numbers are the reference's.
PARITY_GATE = {"tol_atol": 1e-3, "tol_rtol": 1e-3, "tol_slack": 1.5,
               "note": "err_kernel <= err_baseline * tol_slack and allclose(atol, rtol); errors vs an fp64 oracle"}
LENGTH_CHANGE_GATE = {"correct_err_max": 1e-2, "discriminant_min": 1.0,
                      "note": "capture at length N, replay at M: answer must be M's, and N's answer must differ"}

# ``num_splits: None`` means "about two blocks per SM": ceil(2 * SMs / heads), at most 64.
ATTN_CONFIGS: dict[str, Any] = {"split": {"BLOCK_N": 128, "num_warps": 4}, "combine": {"BLOCK_D": 128, "num_warps": 4},
                                "num_splits": None}
_INT32_SPAN = 1 << 31
_KERNEL_BACKENDS = ("auto", "cuda", "triton")  # "triton" is what the reference calls "the kernel"
_SPLIT_CAP = 64

Rule = tuple[Callable[[], bool], type, str]


def _enforce(rules: Iterable[Rule]) -> None:
    """Raise the error of the first rule whose predicate is false.  Predicates are thunks, so a later rule may rely
    on what an earlier one established."""
    for holds, error, text in rules:
        if not holds():
            raise error(text)


def _pow2(n: int) -> bool:
    return n > 0 and n & (n - 1) == 0


def attn_decode_available() -> bool:
    return _cabi.available() and torch.cuda.is_available()


def merged_config(config: dict[str, Any] | None = None) -> dict[str, Any]:
    """A private copy of ``ATTN_CONFIGS`` with ``config`` laid over it (the per-kernel blocks merge key by key)."""
    out = copy.deepcopy(ATTN_CONFIGS)
    for key, new in (config or {}).items():
        if isinstance(new, dict) and isinstance(out.get(key), dict):
            out[key] |= new
        else:
            out[key] = new
    return out


def _sm_count(device: Any) -> int:
    if not torch.cuda.is_available():
        return 0
    try:
        return int(torch.cuda.get_device_properties(0 if device is None else device).multi_processor_count)
    except Exception:  # noqa: BLE001 - a device that cannot be queried counts as "unknown"
        return 0


def resolve_num_splits(num_splits: int | None, *, heads: int, device: Any = None) -> int:
    if num_splits is None:
        sms = _sm_count(device)
        return min(_SPLIT_CAP, max(1, math.ceil(2 * sms / max(1, int(heads))))) if sms else 1
    if int(num_splits) < 1:
        raise ValueError("num_splits 必须 >= 1 (got %r)" % (num_splits,))
    return int(num_splits)


def launch_plan(*, heads: int, head_dim: int, num_splits: int, block_n: int = 128,
                block_d: int | None = None) -> dict[str, Any]:
    """Grid and partial-result shapes of one call, computed on the host alone."""
    width = int(head_dim if block_d is None or not block_d else block_d)
    _enforce((
        (lambda: heads >= 1 and head_dim >= 1, ValueError, "heads 与 head_dim 必须为正 (positive)"),
        (lambda: num_splits >= 1, ValueError, "num_splits 必须 >= 1"),
        (lambda: _pow2(int(head_dim)), ValueError, "head_dim 必须是 2 的幂 (power of two), got %r" % (head_dim,)),
        (lambda: _pow2(int(block_n)), ValueError, "BLOCK_N 必须是 2 的幂 (power of two), got %r" % (block_n,)),
        (lambda: width >= head_dim, ValueError, "BLOCK_D 不能小于 head_dim"),
    ))
    h, d, s = int(heads), int(head_dim), int(num_splits)
    split = {"grid": (s, h), "threads": 128, "partial_shape": (h, s, d + 2), "dtype": "float32"}
    merge = {"fused_into": "split (last block per head)", "out_shape": (1, h, 1, d)}
    return {"heads": h, "head_dim": d, "num_splits": s, "BLOCK_N": int(block_n), "BLOCK_D": width, "kernel_count": 1,
            "split": split, "combine": merge}


def judge_length_change(*, correct_err: float, stale_err: float, gate: dict[str, Any] | None = None) -> dict[str, Any]:
    """Verdict of a capture-at-N / replay-at-M experiment.  The experiment only says something when the stale answer
    (length N's) is far from the right one; otherwise it is INCONCLUSIVE whatever the error."""
    gate = dict(LENGTH_CHANGE_GATE if gate is None else gate)
    correct_err, stale_err = float(correct_err), float(stale_err)
    discriminating = stale_err >= float(gate["discriminant_min"])
    if not discriminating:
        verdict = "INCONCLUSIVE"
    else:
        verdict = "PASS" if correct_err < float(gate["correct_err_max"]) else "FAIL"
    return {"verdict": verdict, "correct_err": correct_err, "stale_err": stale_err, "discriminating": discriminating, "gate": gate}


# ---------------------------------------------------------------------------------------------------------------
# operands
# ---------------------------------------------------------------------------------------------------------------
def _length_scalar(filled_len: Any, *, device: Any, capacity: int) -> Any:
    """The filled length as a one-element int32 tensor on ``device``.  A tensor is taken as it is (its value is not
    read on the host: that would break graph capture); an int is range-checked and uploaded."""
    if torch.is_tensor(filled_len):
        t = filled_len
        _enforce((
            (lambda: t.numel() == 1, ValueError, "filled_len 张量必须是 1 个元素 (one element), got %d" % int(t.numel())),
            (lambda: t.dtype == torch.int32, ValueError, "filled_len 张量必须是 int32, got %s" % t.dtype),
            (lambda: t.device == device, ValueError, "filled_len 与 k/v 不在同一设备: %s vs %s" % (t.device, device)),
        ))
        return t.reshape(1)
    if type(filled_len) is not int:  # bool and numpy integers are refused like the reference does
        raise ValueError("filled_len 必须为 int 或单元素 int32 张量")
    if not 0 <= filled_len <= capacity:
        raise ValueError("filled_len=%d 必须在 [0, %d] 内" % (filled_len, capacity))
    return torch.full((1,), filled_len, dtype=torch.int32, device=device)


def _four_dim_rules(named: dict[str, Any]) -> list[Rule]:
    rules: list[Rule] = []
    for name, t in named.items():
        rules += [
            (lambda t=t: torch.is_tensor(t), TypeError, "%s 必须是张量 (a tensor)" % name),
            (lambda t=t: t.dim() == 4, ValueError, "%s 必须是 4 维 (1,H,S,D), got %s" % (name, tuple(getattr(t, "shape", ()))),),
            (lambda t=t: t.stride(-1) == 1, ValueError, "%s 的最后一维必须连续 (unit stride)" % name),
            (lambda t=t: t.numel() < _INT32_SPAN, ValueError, "%s 的元素数超过 int32 偏移上限" % name),
        ]
    return rules


@dataclass
class _Call:
    """Everything one launch needs besides the key/value pointers."""

    query: Any        # (H, D) contiguous fp16
    heads: int
    head_dim: int
    capacity: int     # positions the cache holds
    head_stride: int  # elements between heads of the key/value arrays
    filled: Any
    splits: int
    scale: float
    out: Any
    scratch: Any

    @classmethod
    def prepare(cls, q: Any, keys: Any, filled_len: Any, cfg: dict[str, Any], scale: float | None) -> "_Call":
        heads, capacity, head_dim = (int(n) for n in keys.shape[1:])
        query = q.reshape(heads, head_dim)
        query = query if query.is_contiguous() else query.contiguous()
        splits = resolve_num_splits(cfg.get("num_splits"), heads=heads, device=keys.device)
        launch_plan(heads=heads, head_dim=head_dim, num_splits=splits, block_n=int(cfg["split"]["BLOCK_N"]))
        return cls(query=query, heads=heads, head_dim=head_dim, capacity=capacity, head_stride=int(keys.stride(1)),
                   filled=_length_scalar(filled_len, device=q.device, capacity=capacity), splits=splits,
                   scale=1.0 / math.sqrt(head_dim) if scale is None else float(scale),
                   out=torch.empty((1, heads, 1, head_dim), dtype=q.dtype, device=q.device),
                   scratch=_workspace(q.device, heads, head_dim, splits))

    def tail(self) -> tuple:
        """Arguments every attention entry point ends with."""
        return (self.heads, self.capacity, self.head_dim, self.splits, self.scale, _cabi.ptr(self.scratch), None,
                _cabi.current_stream(self.query.device))


_WORKSPACES: dict[tuple, Any] = {}


def _workspace(device: Any, heads: int, head_dim: int, num_splits: int) -> Any:
    """Partials and arrival counters of one (device, shape): zeroed once, and every launch leaves the counters at zero.
    Launches that share it must be ordered on the GPU (one stream)."""
    key = (str(device), heads, head_dim, num_splits)
    if key not in _WORKSPACES:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("attention workspace must be created before capture: call warm() first")
        size = int(_cabi.lib().lemoq_attn_workspace_bytes(heads, head_dim, num_splits))
        _WORKSPACES[key] = torch.zeros(size, dtype=torch.uint8, device=device)
    return _WORKSPACES[key]


def _check_backend(backend: str) -> None:
    if backend == "oracle":
        raise RuntimeError("backend='oracle' is not part of this package: the CPU oracle lives in the test "
                           "infrastructure, the product has the CUDA kernel only")
    if backend not in _KERNEL_BACKENDS:
        raise ValueError("unknown backend %r" % (backend,))
    if not attn_decode_available():
        raise RuntimeError("attn_decode 的 kernel 路径不可用: %s" % (_cabi.unavailable_reason() or "no CUDA device"))


# ---------------------------------------------------------------------------------------------------------------
# the two operators
# ---------------------------------------------------------------------------------------------------------------
def attn_decode_forward(q: Any, k: Any, v: Any, filled_len: Any, *, config: dict[str, Any] | None = None,
                        backend: str = "auto", scale: float | None = None) -> Any:
    """``q (1,H,1,D)`` against the whole static fp16 cache ``k, v (1,H,max_len,D)`` -> ``(1,H,1,D)`` fp16.
    Only positions ``[0, filled_len)`` are read; ``filled_len`` is an int or a one-element int32 device tensor."""
    cfg = merged_config(config)
    _enforce(_four_dim_rules({"q": q, "k": k, "v": v}) + [
        (lambda: q.shape[0] == 1 and q.shape[2] == 1, NotImplementedError, "attn_decode 只处理 batch=1 / q_len=1"),
        (lambda: k.shape == v.shape, ValueError, "k 与 v 形状必须相同 (same shape)"),
        (lambda: k.shape[0] == 1 and k.shape[3] == q.shape[3], ValueError, "k/v 必须为 batch=1 且 head_dim 与 q 相同"),
        (lambda: q.device == k.device == v.device, ValueError, "q/k/v 必须在同一设备 (one device)"),
        (lambda: k.stride(2) == k.shape[3] and v.stride(2) == v.shape[3], ValueError, "k/v 的序列 stride 必须等于 head_dim"),
        (lambda: k.stride(1) == v.stride(1) and k.stride(1) >= k.shape[2] * k.shape[3], ValueError,
         "k/v 必须有相同且不重叠的 head stride"),
        (lambda: k.shape[1] == q.shape[1], NotImplementedError,
         "attn_decode 不做 GQA: k has %d heads, q has %d" % (int(k.shape[1]), int(q.shape[1]))),
        (lambda: q.dtype == k.dtype == v.dtype, ValueError, "q 与 k/v dtype 必须相同"),
    ])
    _check_backend(backend)
    if q.dtype != torch.float16:
        raise ValueError("attention kernel 仅支持 fp16")
    _cabi.require_cuda(q, k, v, what="attn_decode_forward")
    call = _Call.prepare(q, k, filled_len, cfg, scale)
    _cabi.call("lemoq_attn_decode_fp16", _cabi.ptr(call.query), _cabi.ptr(k), _cabi.ptr(v), call.head_stride,
               _cabi.ptr(call.filled), _cabi.ptr(call.out), *call.tail())
    return call.out


def attn_decode_forward_int8(q: Any, k_codes: Any, k_scale: Any, v_codes: Any, v_scale: Any, filled_len: Any, *,
                             config: dict[str, Any] | None = None, scale: float | None = None) -> Any:
    """The same contract on the int8 mirror: codes ``(1,H,S,D)`` int8, one fp16 scale per position ``(1,H,S)``.
    ``score_t = qk_scale * (q . kc_t) * ks_t`` and ``acc += (p_t * vs_t) * vc_t``."""
    cfg = merged_config(config)
    codes = {"k_codes": k_codes, "v_codes": v_codes}
    scales = {"k_scale": k_scale, "v_scale": v_scale}
    rules: list[Rule] = []
    for name, t in {"q": q, **codes}.items():
        rules += [(lambda t=t: torch.is_tensor(t) and t.dim() == 4, ValueError, "%s 必须是 4 维张量" % name),
                  (lambda t=t: t.stride(-1) == 1, ValueError, "%s 的最后一维必须连续" % name)]
    for name, t in scales.items():
        rules.append((lambda t=t: torch.is_tensor(t) and t.dim() == 3, ValueError, "%s 必须是 3 维 (1,H,S)" % name))
    rules += [
        (lambda: all(t.dtype == torch.int8 for t in codes.values()), ValueError, "codes 必须 int8"),
        (lambda: all(t.dtype == torch.float16 for t in scales.values()), ValueError, "scale 必须 fp16"),
        (lambda: q.shape[0] == 1 and q.shape[2] == 1, NotImplementedError, "int8 attention 只处理 batch=1 / q_len=1"),
        (lambda: k_codes.shape == v_codes.shape and q.shape[1] == k_codes.shape[1], ValueError,
         "k/v codes 形状必须一致且头数与 q 相同"),
        (lambda: all(tuple(t.shape) == tuple(k_codes.shape[:3]) for t in scales.values()), ValueError, "scale 必须是 (1,H,S)"),
        (lambda: q.is_cuda and k_codes.is_cuda, RuntimeError, "int8 attention 需要 CUDA"),
        (lambda: int(k_codes.shape[3]) >= 2 and _pow2(int(k_codes.shape[3])), ValueError, "head_dim 必须是 2 的幂"),
        (lambda: q.dtype == torch.float16, ValueError, "attention kernel 仅支持 fp16"),
        (lambda: k_codes.stride(2) == v_codes.stride(2) == k_codes.shape[3] and k_codes.stride(1) == v_codes.stride(1),
         ValueError, "k/v codes 的布局必须是 (1,H,S,D) 行连续且 head stride 相同"),
        (lambda: all(t.is_contiguous() for t in scales.values()), ValueError, "scale 必须连续"),
    ]
    _enforce(rules)
    _check_backend("auto")
    call = _Call.prepare(q, k_codes, filled_len, cfg, scale)
    _cabi.call("lemoq_attn_decode_int8", _cabi.ptr(call.query), _cabi.ptr(k_codes), _cabi.ptr(k_scale), _cabi.ptr(v_codes),
               _cabi.ptr(v_scale), call.head_stride, _cabi.ptr(call.filled), _cabi.ptr(call.out), *call.tail())
    return call.out


def warm(*, heads: int, head_dim: int, kv_len: int, filled: int | None = None, dtype: Any = None, device: Any = None,
         config: dict[str, Any] | None = None) -> dict[str, Any]:
    """One real launch before capture.  The kernels are precompiled, so all this buys is the per-shape workspace,
    which must not be allocated during capture."""
    dtype = dtype or torch.float16
    device = torch.device(device or "cuda")
    length = kv_len if filled is None else filled
    zeros = lambda positions: torch.zeros((1, heads, positions, head_dim), dtype=dtype, device=device)  # noqa: E731
    attn_decode_forward(zeros(1), zeros(kv_len), zeros(kv_len), torch.full((1,), int(length), dtype=torch.int32, device=device),
                        config=config)
    torch.cuda.synchronize()
    cfg = merged_config(config)
    return {"heads": int(heads), "head_dim": int(head_dim), "kv_len": int(kv_len), "filled": int(length), "dtype": str(dtype),
            "device": str(device), "BLOCK_N": int(cfg["split"]["BLOCK_N"]),
            "num_splits": resolve_num_splits(cfg.get("num_splits"), heads=int(heads), device=device)}


# ---------------------------------------------------------------------------------------------------------------
# wiring into the OLMoE attention modules (per instance, reversible)
# ---------------------------------------------------------------------------------------------------------------
_ATTENTION_PARTS = ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "num_heads", "head_dim")
_INSTALLED = ("_lemoq_original_forward", "_lemoq_attn_config", "_lemoq_attn_backend")


def _is_olmoe_attention(module: Any) -> bool:
    return all(hasattr(module, part) for part in _ATTENTION_PARTS)


def _attention_modules(model: Any) -> list[Any]:
    """The attention module of every decoder layer, in layer order; for a model without ``model.layers`` every
    sub-module that looks like one."""
    decoder_layers = getattr(getattr(model, "model", None), "layers", None) or ()
    candidates = [getattr(layer, "self_attn", None) for layer in decoder_layers]
    picked = [m for m in candidates if m is not None and _is_olmoe_attention(m)]
    if not picked:
        picked = [m for m in model.modules() if _is_olmoe_attention(m)]
    unique: list[Any] = []
    for module in picked:
        if not any(module is seen for seen in unique):
            unique.append(module)
    return unique


def _kv_int8_bufs_stale(module: Any, past_key_values: Any) -> bool:
    """The int8 mirror belongs to the cache OBJECT it was built from: the same object refilled keeps it, another
    object (or a collected one) does not."""
    source = getattr(module, "_lemoq_kv_int8_src_cache_ref", None)
    if getattr(module, "_lemoq_kv_int8_bufs", None) is None or source is None:
        return True
    return source() is not past_key_values


def _filled_len_of(past_key_values: Any) -> Any:
    return getattr(past_key_values, "_lemoq_filled_len", None) if past_key_values is not None else None


def _project_qkv(module: Any, x: Any) -> tuple[Any, Any, Any]:
    """q and k normalised over the full projection row, v plain; one stacked GEMV when it is installed and on."""
    from lemoq.kernels.packed_qkv import packed_qkv_enabled

    stacked = getattr(module, "_lemoq_packed_qkv", None)
    if stacked is not None and packed_qkv_enabled():
        q, k, v = (t.contiguous() for t in stacked.project(x))
    else:
        q, k, v = module.q_proj(x), module.k_proj(x), module.v_proj(x)
    q, k = module.q_norm(q), module.k_norm(k)
    limit = getattr(module.config, "clip_qkv", None)
    if limit is not None:
        for t in (q, k, v):
            t.clamp_(min=-limit, max=limit)
    return q, k, v


def _store_row(module: Any, cache: Any, k_row: Any, v_row: Any, cos: Any, sin: Any, slot: Any) -> tuple[Any, Any]:
    """Write this step's key/value row into the fp16 cache; returns the arrays attention reads."""
    from lemoq.kernels.fusion_switches import fusion_enabled
    from lemoq.kernels.kv_direct import kv_direct_write, kv_direct_write_applicable

    if cache is None:
        return k_row, v_row
    layer = cache.layers[module.layer_idx]
    if fusion_enabled("kv_direct_write") and kv_direct_write_applicable(layer, k_row, v_row):
        kv_direct_write(layer, k_row, v_row, slot)
        return layer.keys, layer.values
    return cache.update(k_row, v_row, module.layer_idx, {"sin": sin, "cos": cos, "cache_position": slot})


def _attend_int8(module: Any, cache: Any, q: Any, k_row: Any, v_row: Any, slot: Any, filled: Any) -> Any:
    """Quantise the new row into the int8 mirror (built on first use, outside capture) and attend over the mirror.
    Returns None when the row's shape is outside what the int8 kernels take."""
    from lemoq.kernels.kv_int8 import kv_int8_cache_write, kv_int8_init_buffers, kv_int8_rows_applicable

    k_row, v_row = k_row.contiguous(), v_row.contiguous()
    if not kv_int8_rows_applicable(k_row, v_row):
        return None
    if _kv_int8_bufs_stale(module, cache):
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("kv_int8 的 buffer 初始化不能发生在 capture 里 (run an eager warm-up step first)")
        layer = cache.layers[module.layer_idx]
        module._lemoq_kv_int8_bufs = kv_int8_init_buffers(layer.keys, layer.values, filled=None)
        module._lemoq_kv_int8_src_cache_ref = weakref.ref(cache)
    mirror = module._lemoq_kv_int8_bufs
    kv_int8_cache_write(mirror, k_row, v_row, slot)
    module._lemoq_kv_int8_runs = getattr(module, "_lemoq_kv_int8_runs", 0) + 1
    return attn_decode_forward_int8(q, mirror["kc"], mirror["ks"], mirror["vc"], mirror["vs"], filled, config=module._lemoq_attn_config)


def _decode_forward_impl(self: Any, hidden_states: Any, attention_mask: Any = None, position_ids: Any = None,
                         past_key_values: Any = None, output_attentions: bool = False, use_cache: bool = False,
                         cache_position: Any = None, position_embeddings: Any = None, **kwargs: Any) -> Any:
    """``forward`` of a patched attention module.  A single-token call on a cache that carries a device length runs
    projections -> q/k RMSNorm -> head split -> RoPE -> cache row write (+ int8 mirror) -> split-KV attention over
    ``[0, filled)`` -> o_proj; every other call (prefill, ``output_attentions``, no device length) goes to the module's
    own forward unchanged."""
    from lemoq.kernels.fusion_switches import fusion_enabled
    from lemoq.kernels.rope import _fused_rope_enabled, apply_rotary_pos_emb_fused, rotate_half_reference

    filled = _filled_len_of(past_key_values)
    single_token = hidden_states.shape[1] == 1
    if not single_token or output_attentions or filled is None or position_embeddings is None:
        return self._lemoq_original_forward(
            hidden_states, attention_mask=attention_mask, position_ids=position_ids, past_key_values=past_key_values,
            output_attentions=output_attentions, use_cache=use_cache, cache_position=cache_position,
            position_embeddings=position_embeddings, **kwargs)
    if int(getattr(self, "num_key_value_groups", 1)) != 1:
        raise NotImplementedError("attn_decode 不做 GQA：num_key_value_heads != num_attention_heads")

    batch = int(hidden_states.shape[0])
    by_head = lambda t, heads: t.view(batch, 1, heads, self.head_dim).transpose(1, 2)  # noqa: E731
    q, k_row, v_row = _project_qkv(self, hidden_states)
    q, k_row, v_row = by_head(q, self.num_heads), by_head(k_row, self.num_key_value_heads), by_head(v_row, self.num_key_value_heads)
    cos, sin = position_embeddings
    rotate = apply_rotary_pos_emb_fused if _fused_rope_enabled() else rotate_half_reference
    q, k_row = rotate(q, k_row, cos, sin)

    keys, values = _store_row(self, past_key_values, k_row, v_row, cos, sin, cache_position)
    mixed = _attend_int8(self, past_key_values, q, k_row, v_row, cache_position, filled) if fusion_enabled("kv_int8") else None
    if mixed is None:
        mixed = attn_decode_forward(q, keys, values, filled, config=self._lemoq_attn_config, backend=self._lemoq_attn_backend)
    self._lemoq_decode_calls += 1
    return self.o_proj(mixed.transpose(1, 2).contiguous().reshape(batch, 1, self.hidden_size)), None


def replace_attention_cores(model: Any, *, backend: str = "cuda", config: dict[str, Any] | None = None) -> int:
    """Give every OLMoE attention module the decode-kernel ``forward`` as an instance attribute; the module's own
    forward stays on ``_lemoq_original_forward``.  Returns the number of modules patched."""
    if backend == "oracle" or backend not in _KERNEL_BACKENDS:
        _check_backend(backend)  # raises: the oracle is test infrastructure, anything else is unknown
    modules = _attention_modules(model)
    if not modules:
        raise RuntimeError("没有找到任何 OLMoE attention 模块 (no OLMoE attention module found)")
    for module in modules:
        module.__dict__.setdefault("_lemoq_original_forward", module.forward)
        module._lemoq_attn_backend = backend if backend == "triton" else "cuda"
        module._lemoq_attn_config = merged_config(config)
        module._lemoq_decode_calls = 0
        module.forward = types.MethodType(_decode_forward_impl, module)
    return len(modules)


def _patched(model: Any) -> list[Any]:
    return [m for m in _attention_modules(model) if hasattr(m, "_lemoq_original_forward")]


def attention_cores_replaced(model: Any) -> int:
    return len(_patched(model))


def _total(model: Any, counter: str) -> int:
    return sum(int(getattr(m, counter, 0)) for m in _attention_modules(model))


def attention_int8_runs(model: Any) -> int:
    return _total(model, "_lemoq_kv_int8_runs")


def decode_call_count(model: Any) -> int:
    return _total(model, "_lemoq_decode_calls")


def restore_attention_cores(model: Any) -> int:
    modules = _patched(model)
    for module in modules:
        module.forward = module._lemoq_original_forward
        for name in _INSTALLED:
            if hasattr(module, name):
                delattr(module, name)
    return len(modules)
