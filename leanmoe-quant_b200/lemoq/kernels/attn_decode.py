"""Split-KV decode attention: host logic around the CUDA kernels
(reference: src/lemoq/kernels/attn_decode.py).

Two kernels' worth of work in ONE launch: per-split online softmax partials and the
deterministic fixed-order merge (done by the last block of each head).  The filled length is
read from device memory, so the launch shape is static and a captured graph serves every step.
fp16 K/V and the int8 mirror (scales folded into scores / weights) are both built.
"""

from __future__ import annotations

import math
import types
import weakref
from typing import Any

import torch

from lemoq import _cabi

__all__ = [
    "PARITY_GATE", "LENGTH_CHANGE_GATE", "ATTN_CONFIGS", "LOG2E", "attn_decode_available", "merged_config",
    "resolve_num_splits", "launch_plan", "attn_decode_forward", "attn_decode_forward_int8", "judge_length_change",
    "warm", "replace_attention_cores", "restore_attention_cores", "attention_cores_replaced", "decode_call_count",
    "attention_int8_runs",
]

LOG2E = 1.4426950408889634

# Frozen before any measurement (same numbers as the reference gates).
PARITY_GATE = {"tol_atol": 1e-3, "tol_rtol": 1e-3, "tol_slack": 1.5,
               "note": "err_kernel <= err_baseline * tol_slack and allclose(atol, rtol); errors vs an fp64 oracle"}
LENGTH_CHANGE_GATE = {"correct_err_max": 1e-2, "discriminant_min": 1.0,
                      "note": "capture at length N, replay at M: answer must be M's, and N's answer must differ"}

# num_splits None -> about two blocks per SM: ceil(2*SM / heads).
ATTN_CONFIGS: dict[str, Any] = {"split": {"BLOCK_N": 128, "num_warps": 4}, "combine": {"BLOCK_D": 128, "num_warps": 4},
                                "num_splits": None}
_MAX_OFFSET = 2**31
_KERNEL_BACKENDS = ("auto", "cuda", "triton")  # "triton" is the reference's name for "the kernel"


def attn_decode_available() -> bool:
    return _cabi.available() and torch.cuda.is_available()


def merged_config(config: dict[str, Any] | None = None) -> dict[str, Any]:
    cfg = {k: dict(v) if isinstance(v, dict) else v for k, v in ATTN_CONFIGS.items()}
    for key, value in (config or {}).items():
        if isinstance(value, dict) and isinstance(cfg.get(key), dict):
            cfg[key].update(value)
        else:
            cfg[key] = value
    return cfg


def resolve_num_splits(num_splits: int | None, *, heads: int, device: Any = None) -> int:
    if num_splits is not None:
        if int(num_splits) < 1:
            raise ValueError("num_splits 必须 >= 1")
        return int(num_splits)
    sm = None
    if torch.cuda.is_available():
        try:
            sm = int(torch.cuda.get_device_properties(device if device is not None else 0).multi_processor_count)
        except Exception:  # noqa: BLE001
            sm = None
    if not sm:
        return 1
    return max(1, min(64, -(-2 * sm // max(1, int(heads)))))


def launch_plan(*, heads: int, head_dim: int, num_splits: int, block_n: int = 128,
                block_d: int | None = None) -> dict[str, Any]:
    """Grid and workspace shapes, computed without touching the GPU."""
    if heads < 1 or head_dim < 1:
        raise ValueError("heads 与 head_dim 必须为正")
    if block_n < 1 or block_n & (block_n - 1):
        raise ValueError("BLOCK_N 必须是 2 的幂，得到 %r" % (block_n,))
    if head_dim & (head_dim - 1):
        raise ValueError("head_dim 必须是 2 的幂，得到 %r" % (head_dim,))
    if num_splits < 1:
        raise ValueError("num_splits 必须 >= 1")
    block_d = int(block_d or head_dim)
    if block_d < head_dim:
        raise ValueError("BLOCK_D 不能小于 head_dim")
    return {
        "heads": int(heads), "head_dim": int(head_dim), "num_splits": int(num_splits), "BLOCK_N": int(block_n),
        "BLOCK_D": block_d, "kernel_count": 1,
        "split": {"grid": (int(num_splits), int(heads)), "threads": 128,
                  "partial_shape": (int(heads), int(num_splits), int(head_dim) + 2), "dtype": "float32"},
        "combine": {"fused_into": "split (last block per head)", "out_shape": (1, int(heads), 1, int(head_dim))},
    }


def judge_length_change(*, correct_err: float, stale_err: float, gate: dict[str, Any] | None = None) -> dict[str, Any]:
    gate = LENGTH_CHANGE_GATE if gate is None else gate
    discriminating = float(stale_err) >= float(gate["discriminant_min"])
    correct = float(correct_err) < float(gate["correct_err_max"])
    verdict = "INCONCLUSIVE" if not discriminating else ("PASS" if correct else "FAIL")
    return {"verdict": verdict, "correct_err": float(correct_err), "stale_err": float(stale_err),
            "discriminating": bool(discriminating), "gate": dict(gate)}


def _filled_tensor(filled_len: Any, *, device: Any, seq_len: int) -> Any:
    if torch.is_tensor(filled_len):
        if filled_len.numel() != 1:
            raise ValueError("filled_len 张量必须是 1 个元素，得到 %d" % int(filled_len.numel()))
        if filled_len.dtype != torch.int32:
            raise ValueError("filled_len 张量必须是 int32，得到 %s" % filled_len.dtype)
        if filled_len.device != device:
            raise ValueError("filled_len 与 k/v 不在同一设备：%s vs %s" % (filled_len.device, device))
        return filled_len.reshape(1)
    if type(filled_len) is not int:
        raise ValueError("filled_len 必须为 int 或单元素 int32 张量")
    if filled_len < 0 or filled_len > seq_len:
        raise ValueError("filled_len=%d 必须在 [0, %d] 内" % (filled_len, seq_len))
    return torch.full((1,), int(filled_len), dtype=torch.int32, device=device)


_WORKSPACES: dict[tuple, Any] = {}


def _workspace(device: Any, heads: int, head_dim: int, num_splits: int) -> Any:
    """Zero-initialised once per (device, shape); every launch leaves the counters at zero.
    Launches that share it must be ordered on the GPU (one stream)."""
    key = (str(device), heads, head_dim, num_splits)
    ws = _WORKSPACES.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("attention workspace must be created before capture: call warm() first")
        nbytes = int(_cabi.lib().lemoq_attn_workspace_bytes(heads, head_dim, num_splits))
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def _check_backend(backend: str) -> None:
    if backend == "oracle":
        raise RuntimeError("backend='oracle' is not part of this package: the CPU oracle lives in the test "
                           "infrastructure, the product has the CUDA kernel only")
    if backend not in _KERNEL_BACKENDS:
        raise ValueError("unknown backend %r" % (backend,))
    if not attn_decode_available():
        raise RuntimeError("attn_decode 的 kernel 路径不可用: %s" % (_cabi.unavailable_reason() or "no CUDA device"))


def attn_decode_forward(q: Any, k: Any, v: Any, filled_len: Any, *, config: dict[str, Any] | None = None,
                        backend: str = "auto", scale: float | None = None) -> Any:
    """``q (1,H,1,D)`` + the whole static fp16 cache ``k/v (1,H,max_len,D)`` -> ``(1,H,1,D)`` fp16.
    Only ``[0, filled_len)`` is read; ``filled_len`` is an int or a one-element int32 device tensor."""
    cfg = merged_config(config)
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        if not torch.is_tensor(tensor):
            raise TypeError("%s 必须是张量" % name)
        if tensor.dim() != 4:
            raise ValueError("%s 必须是 4 维，得到 %s" % (name, tuple(tensor.shape)))
        if tensor.stride(-1) != 1:
            raise ValueError("%s 的最后一维必须连续" % name)
        if tensor.numel() >= _MAX_OFFSET:
            raise ValueError("%s 的元素数超过 int32 偏移上限" % name)
    if int(q.shape[2]) != 1 or int(q.shape[0]) != 1:
        raise NotImplementedError("attn_decode 只处理 batch=1 / q_len=1")
    if tuple(k.shape) != tuple(v.shape):
        raise ValueError("k 与 v 形状必须相同")
    if int(k.shape[0]) != 1 or int(k.shape[3]) != int(q.shape[3]):
        raise ValueError("k/v 必须为 batch=1 且 head_dim 与 q 相同")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q/k/v 必须在同一设备")
    if k.stride(2) != k.shape[3] or v.stride(2) != v.shape[3]:
        raise ValueError("k/v 的序列 stride 必须等于 head_dim")
    if k.stride(1) != v.stride(1) or k.stride(1) < k.shape[2] * k.shape[3]:
        raise ValueError("k/v 必须有相同且不重叠的 head stride")
    if int(k.shape[1]) != int(q.shape[1]):
        raise NotImplementedError("attn_decode 不做 GQA：k 的 head 数 %d != q 的 %d" % (int(k.shape[1]), int(q.shape[1])))
    if k.dtype != v.dtype or q.dtype != k.dtype:
        raise ValueError("q 与 k/v dtype 必须相同")
    _check_backend(backend)
    if q.dtype != torch.float16:
        raise ValueError("attention kernel 仅支持 fp16")
    _cabi.require_cuda(q, k, v, what="attn_decode_forward")
    heads, head_dim, seq_len = int(q.shape[1]), int(q.shape[3]), int(k.shape[2])
    filled = _filled_tensor(filled_len, device=q.device, seq_len=seq_len)
    num_splits = resolve_num_splits(cfg.get("num_splits"), heads=heads, device=k.device)
    launch_plan(heads=heads, head_dim=head_dim, num_splits=num_splits, block_n=int(cfg["split"]["BLOCK_N"]))
    qc = q.reshape(heads, head_dim)
    if not qc.is_contiguous():
        qc = qc.contiguous()
    out = torch.empty((1, heads, 1, head_dim), dtype=q.dtype, device=q.device)
    ws = _workspace(q.device, heads, head_dim, num_splits)
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    _cabi.call("lemoq_attn_decode_fp16", _cabi.ptr(qc), _cabi.ptr(k), _cabi.ptr(v), int(k.stride(1)), _cabi.ptr(filled),
               _cabi.ptr(out), heads, seq_len, head_dim, num_splits, sc, _cabi.ptr(ws), None,
               _cabi.current_stream(q.device))
    return out


def attn_decode_forward_int8(q: Any, k_codes: Any, k_scale: Any, v_codes: Any, v_scale: Any, filled_len: Any, *,
                             config: dict[str, Any] | None = None, scale: float | None = None) -> Any:
    """Same contract on the int8 mirror: ``k_codes/v_codes (1,H,S,D)`` int8 and per-token scales
    ``(1,H,S)`` fp16; ``score_t = qk_scale * (q . c_t) * ks_t`` and ``acc += (p_t * vs_t) * cv_t``."""
    cfg = merged_config(config)
    for name, tensor in (("q", q), ("k_codes", k_codes), ("v_codes", v_codes)):
        if not torch.is_tensor(tensor) or tensor.dim() != 4:
            raise ValueError("%s 必须是 4 维张量" % name)
        if tensor.stride(-1) != 1:
            raise ValueError("%s 的最后一维必须连续" % name)
    for name, tensor in (("k_scale", k_scale), ("v_scale", v_scale)):
        if not torch.is_tensor(tensor) or tensor.dim() != 3:
            raise ValueError("%s 必须是 3 维 (1,H,S)" % name)
    if k_codes.dtype != torch.int8 or v_codes.dtype != torch.int8:
        raise ValueError("codes 必须 int8")
    if k_scale.dtype != torch.float16 or v_scale.dtype != torch.float16:
        raise ValueError("scale 必须 fp16")
    if int(q.shape[2]) != 1 or int(q.shape[0]) != 1:
        raise NotImplementedError("int8 attention 只处理 batch=1 / q_len=1")
    heads, seq_len, head_dim = int(k_codes.shape[1]), int(k_codes.shape[2]), int(k_codes.shape[3])
    if tuple(k_codes.shape) != tuple(v_codes.shape) or int(q.shape[1]) != heads:
        raise ValueError("k/v codes 形状必须一致且头数与 q 相同")
    if tuple(k_scale.shape) != (1, heads, seq_len) or tuple(v_scale.shape) != (1, heads, seq_len):
        raise ValueError("scale 必须是 (1,H,S)")
    if not (k_codes.is_cuda and q.is_cuda):
        raise RuntimeError("int8 attention 需要 CUDA")
    if int(head_dim - 1) & int(head_dim) or head_dim < 2:
        raise ValueError("head_dim 必须是 2 的幂")
    if q.dtype != torch.float16:
        raise ValueError("attention kernel 仅支持 fp16")
    if k_codes.stride(2) != head_dim or v_codes.stride(2) != head_dim or k_codes.stride(1) != v_codes.stride(1):
        raise ValueError("k/v codes 的布局必须是 (1,H,S,D) 行连续且 head stride 相同")
    if not (k_scale.is_contiguous() and v_scale.is_contiguous()):
        raise ValueError("scale 必须连续")
    _check_backend("auto")
    filled = _filled_tensor(filled_len, device=q.device, seq_len=seq_len)
    num_splits = resolve_num_splits(cfg.get("num_splits"), heads=heads, device=q.device)
    qc = q.reshape(heads, head_dim)
    if not qc.is_contiguous():
        qc = qc.contiguous()
    out = torch.empty((1, heads, 1, head_dim), dtype=q.dtype, device=q.device)
    ws = _workspace(q.device, heads, head_dim, num_splits)
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    _cabi.call("lemoq_attn_decode_int8", _cabi.ptr(qc), _cabi.ptr(k_codes), _cabi.ptr(k_scale), _cabi.ptr(v_codes),
               _cabi.ptr(v_scale), int(k_codes.stride(1)), _cabi.ptr(filled), _cabi.ptr(out), heads, seq_len, head_dim,
               num_splits, sc, _cabi.ptr(ws), None, _cabi.current_stream(q.device))
    return out


def warm(*, heads: int, head_dim: int, kv_len: int, filled: int | None = None, dtype: Any = None, device: Any = None,
         config: dict[str, Any] | None = None) -> dict[str, Any]:
    """One real launch before capture: creates the per-shape workspace (the kernels themselves are
    precompiled, nothing is JIT-built)."""
    dtype = torch.float16 if dtype is None else dtype
    device = torch.device("cuda" if device is None else device)
    q = torch.zeros((1, heads, 1, head_dim), dtype=dtype, device=device)
    k = torch.zeros((1, heads, kv_len, head_dim), dtype=dtype, device=device)
    v = torch.zeros((1, heads, kv_len, head_dim), dtype=dtype, device=device)
    n = int(filled if filled is not None else kv_len)
    attn_decode_forward(q, k, v, torch.full((1,), n, dtype=torch.int32, device=device), config=config)
    torch.cuda.synchronize()
    cfg = merged_config(config)
    return {"heads": int(heads), "head_dim": int(head_dim), "kv_len": int(kv_len), "filled": n, "dtype": str(dtype),
            "device": str(device),
            "num_splits": resolve_num_splits(cfg.get("num_splits"), heads=int(heads), device=device),
            "BLOCK_N": int(cfg["split"]["BLOCK_N"])}


# ---------------------------------------------------------------------------
# wiring into the OLMoE attention modules (instance-level, reversible)
# ---------------------------------------------------------------------------
def _is_olmoe_attention(module: Any) -> bool:
    needed = ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")
    return all(hasattr(module, n) for n in needed) and hasattr(module, "num_heads") and hasattr(module, "head_dim")


def _attention_modules(model: Any) -> list[Any]:
    found: list[Any] = []
    layers = getattr(getattr(model, "model", None), "layers", None)
    if layers is not None:
        for layer in layers:
            attn = getattr(layer, "self_attn", None)
            if attn is not None and _is_olmoe_attention(attn) and attn not in found:
                found.append(attn)
    if found:
        return found
    for module in model.modules():
        if _is_olmoe_attention(module) and module not in found:
            found.append(module)
    return found


def _kv_int8_bufs_stale(module: Any, past_key_values: Any) -> bool:
    """The mirror is tied to the cache OBJECT it was built from (same object refilled = reuse)."""
    if getattr(module, "_lemoq_kv_int8_bufs", None) is None:
        return True
    ref = getattr(module, "_lemoq_kv_int8_src_cache_ref", None)
    return ref is None or ref() is not past_key_values


def _filled_len_of(past_key_values: Any) -> Any:
    return None if past_key_values is None else getattr(past_key_values, "_lemoq_filled_len", None)


def _decode_forward_impl(self: Any, hidden_states: Any, attention_mask: Any = None, position_ids: Any = None,
                         past_key_values: Any = None, output_attentions: bool = False, use_cache: bool = False,
                         cache_position: Any = None, position_embeddings: Any = None, **kwargs: Any) -> Any:
    """Replacement of the attention module's forward for ``q_len == 1``: projections (packed when
    installed) -> q/k RMSNorm on the full projection rows -> head split -> RoPE -> KV slot write
    (+ int8 mirror write) -> split-KV attention over ``[0, filled)`` -> o_proj.  Any other call
    (prefill, no device length, ``output_attentions``) goes to the module's original forward."""
    from lemoq.kernels.fusion_switches import fusion_enabled
    from lemoq.kernels.packed_qkv import packed_qkv_enabled
    from lemoq.kernels.rope import _fused_rope_enabled, apply_rotary_pos_emb_fused, rotate_half_reference

    original = self._lemoq_original_forward
    filled = _filled_len_of(past_key_values)
    q_len = int(hidden_states.shape[1])
    if output_attentions or q_len != 1 or filled is None or position_embeddings is None:
        return original(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                        past_key_values=past_key_values, output_attentions=output_attentions, use_cache=use_cache,
                        cache_position=cache_position, position_embeddings=position_embeddings, **kwargs)
    if int(getattr(self, "num_key_value_groups", 1)) != 1:
        raise NotImplementedError("attn_decode 不做 GQA：num_key_value_heads != num_attention_heads")

    bsz = int(hidden_states.shape[0])
    packed = getattr(self, "_lemoq_packed_qkv", None)
    if packed is not None and packed_qkv_enabled():
        q_states, k_states, v_states = packed.project(hidden_states)
        query_states, key_states, value_states = self.q_norm(q_states.contiguous()), self.k_norm(k_states.contiguous()), v_states
    else:
        query_states = self.q_norm(self.q_proj(hidden_states))
        key_states = self.k_norm(self.k_proj(hidden_states))
        value_states = self.v_proj(hidden_states)
    clip_qkv = getattr(self.config, "clip_qkv", None)
    if clip_qkv is not None:
        query_states.clamp_(min=-clip_qkv, max=clip_qkv)
        key_states.clamp_(min=-clip_qkv, max=clip_qkv)
        value_states.clamp_(min=-clip_qkv, max=clip_qkv)
    query_states = query_states.view(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
    key_states = key_states.view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
    value_states = value_states.view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)

    cos, sin = position_embeddings
    if _fused_rope_enabled():
        query_states, key_states = apply_rotary_pos_emb_fused(query_states, key_states, cos, sin)
    else:
        query_states, key_states = rotate_half_reference(query_states, key_states, cos, sin)

    new_key, new_value = key_states, value_states
    if past_key_values is not None:
        from lemoq.kernels.kv_direct import kv_direct_write, kv_direct_write_applicable

        layer = past_key_values.layers[self.layer_idx]
        if fusion_enabled("kv_direct_write") and kv_direct_write_applicable(layer, key_states, value_states):
            kv_direct_write(layer, key_states, value_states, cache_position)
            key_states, value_states = layer.keys, layer.values
        else:
            key_states, value_states = past_key_values.update(
                key_states, value_states, self.layer_idx, {"sin": sin, "cos": cos, "cache_position": cache_position})

    kv8 = fusion_enabled("kv_int8")
    if kv8:
        from lemoq.kernels.kv_int8 import kv_int8_rows_applicable

        nk, nv = new_key.contiguous(), new_value.contiguous()
        if not kv_int8_rows_applicable(nk, nv):
            kv8 = False
    if kv8:
        from lemoq.kernels.kv_int8 import kv_int8_cache_write, kv_int8_init_buffers

        if _kv_int8_bufs_stale(self, past_key_values):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("kv_int8 的 buffer 初始化不能发生在 capture 里 (run an eager warm-up step first)")
            layer = past_key_values.layers[self.layer_idx]
            self._lemoq_kv_int8_bufs = kv_int8_init_buffers(layer.keys, layer.values, filled=None)
            self._lemoq_kv_int8_src_cache_ref = weakref.ref(past_key_values)
        bufs = self._lemoq_kv_int8_bufs
        kv_int8_cache_write(bufs, nk, nv, cache_position)
        attn_output = attn_decode_forward_int8(query_states, bufs["kc"], bufs["ks"], bufs["vc"], bufs["vs"], filled,
                                               config=self._lemoq_attn_config)
        self._lemoq_kv_int8_runs = getattr(self, "_lemoq_kv_int8_runs", 0) + 1
    else:
        attn_output = attn_decode_forward(query_states, key_states, value_states, filled,
                                          config=self._lemoq_attn_config, backend=self._lemoq_attn_backend)
    attn_output = attn_output.transpose(1, 2).contiguous().reshape(bsz, q_len, self.hidden_size)
    attn_output = self.o_proj(attn_output)
    self._lemoq_decode_calls += 1
    return attn_output, None


def replace_attention_cores(model: Any, *, backend: str = "cuda", config: dict[str, Any] | None = None) -> int:
    """Swap every OLMoE attention module's ``forward`` for the decode-kernel version (instance
    attribute; the original is kept on ``_lemoq_original_forward``)."""
    if backend == "oracle":
        _check_backend(backend)
    if backend not in _KERNEL_BACKENDS:
        raise ValueError("unknown backend %r" % (backend,))
    patched = 0
    for module in _attention_modules(model):
        if not hasattr(module, "_lemoq_original_forward"):
            module._lemoq_original_forward = module.forward
        module._lemoq_attn_backend = "triton" if backend == "triton" else "cuda"
        module._lemoq_attn_config = merged_config(config)
        module._lemoq_decode_calls = 0
        module.forward = types.MethodType(_decode_forward_impl, module)
        patched += 1
    if not patched:
        raise RuntimeError("没有找到任何 OLMoE attention 模块 (no OLMoE attention module found)")
    return patched


def attention_cores_replaced(model: Any) -> int:
    return sum(1 for m in _attention_modules(model) if hasattr(m, "_lemoq_original_forward"))


def attention_int8_runs(model: Any) -> int:
    return sum(int(getattr(m, "_lemoq_kv_int8_runs", 0)) for m in _attention_modules(model))


def decode_call_count(model: Any) -> int:
    return sum(int(getattr(m, "_lemoq_decode_calls", 0)) for m in _attention_modules(model))


def restore_attention_cores(model: Any) -> int:
    restored = 0
    for module in _attention_modules(model):
        if hasattr(module, "_lemoq_original_forward"):
            module.forward = module._lemoq_original_forward
            for attr in ("_lemoq_original_forward", "_lemoq_attn_config", "_lemoq_attn_backend"):
                try:
                    delattr(module, attr)
                except AttributeError:
                    pass
            restored += 1
    return restored
