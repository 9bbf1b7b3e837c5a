"""Gather-free grouped MoE decode on fp16 expert weights
(reference: src/lemoq/kernels/moe_grouped.py).

``out[n] = sum_i top_w[i] * (Wd[e_i] . act_i)`` with ``act_i = silu(Wg[e_i] . x) * (Wu[e_i] . x)``;
the expert id only enters pointer arithmetic, so shapes are static and the call is graph-safe.
"""

from __future__ import annotations

from typing import Any

import torch

from lemoq import _cabi

__all__ = ["PARITY_GATE", "GROUPED_CONFIGS", "grouped_available", "grouped_moe_forward", "static_moe_forward_grouped",
           "launch_plan", "merged_config", "warm"]

PARITY_GATE = {"tol_atol": 1e-3, "tol_rtol": 1e-3, "tol_slack": 1.5,
               "note": "err_kernel <= err_baseline * tol_slack and allclose(atol, rtol); errors vs an fp64 oracle"}

# Tile description of the CUDA kernels (informational; tuned in the kernel source, not from Python).
# gate_up: one warp per (slot, n) streams the gate row and the up row (4 KB in flight per warp).
# down: one warp owns 2 output rows and walks the K slots with a two-deep prefetch; the K
# activation vectors sit in shared memory.  No split-K, no separate reduction kernels.
GROUPED_CONFIGS: dict[str, dict[str, int]] = {
    "gate_up_act": {"BLOCK_N": 8, "BLOCK_K": 512, "SPLIT_K": 1, "num_warps": 8},
    "down_sum": {"BLOCK_N": 8, "BLOCK_K": 512, "SPLIT_K": 1, "num_warps": 4},
}
_MAX_OFFSET = 2**31


def grouped_available() -> bool:
    return _cabi.available() and torch.cuda.is_available()


def _check_act_fn(act_fn: Any) -> None:
    import torch.nn.functional as F

    if act_fn is None or act_fn is F.silu or getattr(act_fn, "__name__", "") == "silu":
        return
    if type(act_fn).__name__ in ("SiLU", "SiLUActivation"):
        return
    raise NotImplementedError("grouped kernels 融合了 silu；act_fn=%r 不是 silu" % (act_fn,))


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def merged_config(config: dict[str, Any] | None = None) -> dict[str, dict[str, Any]]:
    cfg = {name: dict(values) for name, values in GROUPED_CONFIGS.items()}
    for key, value in (config or {}).items():
        cfg.setdefault(key, {}).update(value)
    return cfg


def launch_plan(fused: Any, *, top_k: int, config: dict[str, Any] | None = None) -> dict[str, Any]:
    """Grids and buffer shapes of the two launches, computed without touching the GPU."""
    gate_up = fused.gate_up
    ffn, hidden = int(gate_up.shape[1]) // 2, int(gate_up.shape[2])
    cfg = merged_config(config)
    ga, ds = cfg["gate_up_act"], cfg["down_sum"]
    return {
        "hidden": hidden, "ffn": ffn, "top_k": top_k,
        "gate_up_act": {"grid": (_cdiv(ffn, int(ga["num_warps"])), top_k, 1), "BLOCK_N": int(ga["BLOCK_N"]),
                        "BLOCK_K": int(ga["BLOCK_K"]), "SPLIT_K": 1, "num_warps": int(ga["num_warps"]),
                        "act_shape": (top_k, ffn), "partial_shape": None},
        "act_combine": None,
        "down_sum": {"grid": (_cdiv(hidden, 2 * int(ds["num_warps"])), 1), "BLOCK_N": int(ds["BLOCK_N"]),
                     "BLOCK_K": int(ds["BLOCK_K"]), "SPLIT_K": 1, "num_warps": int(ds["num_warps"]),
                     "out_shape": (hidden,), "partial_shape": None},
        "out_reduce": None,
        "kernel_count": 2,
    }


def _prepare(x: Any, ids: Any, top_w: Any, dt: Any):
    xf = x.reshape(-1).contiguous()
    if xf.dtype != dt:
        xf = xf.to(dt)
    idx = ids.reshape(-1).contiguous()
    if idx.dtype != torch.int64:
        idx = idx.to(torch.int64)
    wsum = top_w.reshape(-1).contiguous()
    if wsum.dtype != dt:
        wsum = wsum.to(dt)
    return xf, idx, wsum


def grouped_moe_forward(x: Any, fused: Any, ids: Any, top_w: Any, *, config: dict[str, Any] | None = None,
                        backend: str = "auto") -> Any:
    """``(H,)`` hidden state + ``(K,)`` expert ids + ``(K,)`` routing weights -> ``(H,)`` fp16."""
    gate_up, down = fused.gate_up, fused.down
    for name, tensor in (("gate_up", gate_up), ("down", down)):
        if not tensor.is_contiguous():
            raise ValueError("%s 必须连续 (must be contiguous)" % name)
        if tensor.numel() >= _MAX_OFFSET:
            raise ValueError("%s 的元素数超过 int32 偏移上限" % name)
    if backend == "oracle":
        raise RuntimeError("backend='oracle' is not part of this package (the CPU oracle is test infrastructure)")
    if backend not in ("auto", "cuda", "triton"):
        raise ValueError("unknown backend %r" % (backend,))
    if gate_up.dtype != torch.float16:
        raise NotImplementedError("grouped kernel 只支持 fp16 融合权重；得到 gate_up.dtype=%s"
                                  % str(gate_up.dtype).replace("torch.", ""))
    if not grouped_available():
        raise RuntimeError("grouped kernels 不可用: %s" % (_cabi.unavailable_reason() or "no CUDA device (triton-free CUDA path)"))
    xf, idx, wsum = _prepare(x, ids, top_w, gate_up.dtype)
    top_k = int(idx.numel())
    e, ffn, hidden = int(gate_up.shape[0]), int(gate_up.shape[1]) // 2, int(gate_up.shape[2])
    if int(xf.numel()) != hidden:
        raise ValueError("grouped_moe_forward 只处理单 token：x 有 %d 个元素，hidden 是 %d" % (int(xf.numel()), hidden))
    if int(wsum.numel()) != top_k:
        raise ValueError("top_w 的长度 %d 与槽位数 %d 不符" % (int(wsum.numel()), top_k))
    if int(down.shape[2]) != ffn:
        raise ValueError("down 的 ffn 维与 gate_up 不一致")
    _cabi.require_cuda(xf, gate_up, down, idx, wsum, what="grouped_moe_forward")
    act = torch.empty((top_k, ffn), dtype=gate_up.dtype, device=xf.device)
    out = torch.empty((hidden,), dtype=gate_up.dtype, device=xf.device)
    _cabi.call("lemoq_moe_grouped_fp16", _cabi.ptr(xf), _cabi.ptr(gate_up), _cabi.ptr(down), _cabi.ptr(idx),
               _cabi.ptr(wsum), 1, top_k, e, hidden, ffn, _cabi.ptr(act), _cabi.ptr(out), None,
               _cabi.current_stream(xf.device))
    return out


def static_moe_forward_grouped(hidden_states: Any, router_weight: Any, fused: Any, *, top_k: int, norm_topk_prob: bool,
                               act_fn: Any, config: dict[str, Any] | None = None) -> tuple[Any, Any]:
    _check_act_fn(act_fn)
    from lemoq.kernels.moe_static import _route

    shape = tuple(hidden_states.shape)
    x = hidden_states.reshape(-1, shape[-1])
    logits, top_w, top_i = _route(x, router_weight, top_k=top_k, norm_topk_prob=norm_topk_prob)
    out = grouped_moe_forward(x, fused, top_i.reshape(-1), top_w.reshape(-1), config=config)
    return out.reshape(*shape), logits


def warm(fused: Any, *, hidden: int, top_k: int, dtype: Any = None, device: Any = None,
         config: dict[str, Any] | None = None) -> dict[str, Any]:
    dev = device if device is not None else fused.gate_up.device
    dt = dtype or fused.gate_up.dtype
    x = torch.zeros(hidden, dtype=dt, device=dev)
    ids = torch.zeros(top_k, dtype=torch.int64, device=dev)
    wsum = torch.full((top_k,), 1.0 / max(top_k, 1), dtype=dt, device=dev)
    grouped_moe_forward(x, fused, ids, wsum, config=config)
    if getattr(dev, "type", None) == "cuda":
        torch.cuda.synchronize()
    return {"hidden": hidden, "top_k": top_k, "dtype": str(dt), "device": str(dev)}
