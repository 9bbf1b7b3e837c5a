"""``QuantLinear`` and ``quantize_model`` (reference: src/lemoq/quant/linear.py).

A quantised ``nn.Linear``: int8 codes (``packed``) and fp16 per-group scales live in buffers.
Single-token CUDA inputs in ``dequant="fused"`` mode go through the W8 GEMV kernel; everything
else (prefill, multi-token) dequantises the weight and calls ``F.linear`` and is counted as a
fallback, exactly like the reference's separate arm.  Only the canonical scheme is built:
``w8a16``, symmetric, RTN.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

DEQUANT_MODES = ("separate", "fused")
_SCHEMES = {"w8a16": (8, None), "fp16": (None, None)}


def parse_scheme(name: str) -> tuple[int | None, int | None]:
    if name not in _SCHEMES:
        raise NotImplementedError("scheme %r is not built on this path (canonical decode is w8a16); have %s"
                                  % (name, sorted(_SCHEMES)))
    return _SCHEMES[name]


@dataclass
class SchemeSpec:
    name: str = "w8a16"
    weight_bits: int | None = 8
    act_bits: int | None = None
    group_size: int = 128
    targets: tuple[str, ...] = ("attention", "experts", "router")
    keep_lm_head_fp16: bool = True
    symmetric: bool = True
    scheme: str = "rtn"
    dequant: str = "separate"

    def __post_init__(self) -> None:
        if str(self.dequant) not in DEQUANT_MODES:
            raise ValueError("未知 dequant 模式 %r；已实现：%s" % (self.dequant, list(DEQUANT_MODES)))

    @classmethod
    def from_flags(cls, name: str, group_size: int, *, targets: tuple[str, ...] | None = None,
                   keep_lm_head_fp16: bool = True, dequant: str = "separate") -> "SchemeSpec":
        bits, act = parse_scheme(name)
        return cls(name=name, weight_bits=bits, act_bits=act, group_size=group_size,
                   targets=targets or ("attention", "experts", "router"), keep_lm_head_fp16=keep_lm_head_fp16,
                   dequant=str(dequant))

    @property
    def enabled(self) -> bool:
        return self.weight_bits is not None

    def to_dict(self) -> dict[str, Any]:
        return {"scheme": self.name, "weight_bits": self.weight_bits, "act_bits": self.act_bits,
                "group_size": self.group_size, "targets": list(self.targets),
                "keep_lm_head_fp16": self.keep_lm_head_fp16, "symmetric": self.symmetric, "rtn_scheme": self.scheme,
                "dequant": self.dequant, "activation_quantization": "none"}


TARGET_RULES: tuple[tuple[str, str], ...] = (
    (r"^lm_head$", "lm_head"),
    (r"\.self_attn\.", "attention"),
    (r"\.experts\.\d+\.", "experts"),
    (r"\.mlp\.gate$", "router"),
    (r"\.shared_expert", "shared"),
)
_LAYER_RE = re.compile(r"\.layers\.(\d+)\.")


def _layer_index(module_name: str) -> int | None:
    m = _LAYER_RE.search(module_name)
    return int(m.group(1)) if m else None


def classify_linear(module_name: str) -> str | None:
    for pattern, target in TARGET_RULES:
        if re.search(pattern, module_name):
            return target
    return None


def _fused_backend() -> tuple[Any, str | None]:
    from lemoq.kernels import dequant_gemv

    reason = dequant_gemv.unavailable_reason()
    return (dequant_gemv, None) if reason is None else (None, reason)


class QuantLinear(nn.Module):
    """Drop-in for a bias-free or biased ``nn.Linear`` holding W8 weights in buffers."""

    def __init__(self, linear: Any, spec: SchemeSpec, *, name: str = "") -> None:
        from lemoq.quant.rtn import quantize_w8

        super().__init__()
        if spec.weight_bits is None:
            raise ValueError("SchemeSpec.weight_bits 为 None：不该构造 QuantLinear")
        if int(spec.weight_bits) != 8 or not spec.symmetric or spec.scheme != "rtn":
            raise NotImplementedError("QuantLinear: only symmetric 8-bit RTN is built (got bits=%r symmetric=%r scheme=%r)"
                                      % (spec.weight_bits, spec.symmetric, spec.scheme))
        self.spec = spec
        self.name = name
        self.in_features = int(linear.in_features)
        self.out_features = int(linear.out_features)
        self.group_size = int(spec.group_size or 0)
        if self.group_size <= 0 or self.in_features % self.group_size != 0:
            raise NotImplementedError("QuantLinear: in_features=%d 不能被 group_size=%d 整除（本路径不补零）"
                                      % (self.in_features, self.group_size))
        codes, scale = quantize_w8(linear.weight.detach(), self.group_size)
        self.register_buffer("packed", codes.contiguous(), persistent=True)
        self.register_buffer("scale", scale.contiguous(), persistent=True)
        self.register_buffer("zero", None)
        self.register_buffer("bias", linear.bias.detach().clone() if linear.bias is not None else None, persistent=True)
        self.weight_bits = 8
        self.padded_in = self.in_features
        self.n_groups = self.in_features // self.group_size
        self.dequant_mode = str(spec.dequant)
        self._counters: dict[str, Any] = {"separate_calls": 0, "fused_calls": 0, "fallbacks": {}}

    def dequantized_weight(self, dtype: Any = None) -> Any:
        """``(out, in)`` floating weight = codes * fp16 scale (the separate arm's per-call work)."""
        codes = self.packed.to(torch.float32).reshape(self.out_features, self.n_groups, self.group_size)
        w = (codes * self.scale.to(torch.float32).reshape(self.out_features, self.n_groups, 1)).reshape(
            self.out_features, self.in_features)
        return w.to(dtype) if dtype is not None else w

    @property
    def fused_available(self) -> bool:
        return _fused_backend()[0] is not None

    def _fused_fallback_reason(self, x: Any) -> str | None:
        if self.dequant_mode != "fused":
            return "mode_is_separate"
        if not x.is_cuda:
            return "not_cuda"
        if x.dtype != torch.float16:
            return "dtype_unsupported(%s)" % str(x.dtype).replace("torch.", "")
        if x.shape[-1] != self.in_features:
            return "input_width_mismatch(%d!=%d)" % (int(x.shape[-1]), self.in_features)
        if int(x.numel() // max(self.in_features, 1)) != 1:
            return "multi_token"
        backend, reason = _fused_backend()
        return None if backend is not None else (reason or "kernel_unavailable")

    def _fused_forward(self, x: Any) -> Any:
        reason = self._fused_fallback_reason(x)
        if reason is not None:
            fb = self._counters["fallbacks"]
            fb[reason] = fb.get(reason, 0) + 1
            return None
        from lemoq.kernels.dequant_gemv import dequant_gemm_fused

        flat = x.reshape(-1, self.in_features)
        y = dequant_gemm_fused(flat if flat.is_contiguous() else flat.contiguous(), self.packed, self.scale, None,
                               group_size=self.group_size, bits=8, symmetric=True, out_dtype=x.dtype)
        y = y.reshape(*x.shape[:-1], self.out_features)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def forward(self, x: Any) -> Any:
        if self.dequant_mode == "fused":
            fused = self._fused_forward(x)
            if fused is not None:
                self._counters["fused_calls"] += 1
                return fused
        self._counters["separate_calls"] += 1
        w = self.dequantized_weight(dtype=x.dtype)
        return F.linear(x, w, self.bias.to(x.dtype) if self.bias is not None else None)

    def extra_repr(self) -> str:
        return "%d->%d %s group=%d" % (self.in_features, self.out_features, self.spec.name, self.group_size)


@dataclass
class QuantizeReport:
    spec: dict[str, Any]
    replaced: dict[str, int] = field(default_factory=dict)
    skipped: list[str] = field(default_factory=list)
    realized_by_target: dict[str, dict[str, int]] = field(default_factory=dict)
    padding: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {"spec": self.spec, "replaced_per_target": self.replaced,
                "realized_bytes_total": sum(v["total_bytes"] for v in self.realized_by_target.values()),
                "realized_bytes_by_target": self.realized_by_target, "padding": self.padding,
                "skipped_linear_count": len(self.skipped), "skipped_linear_examples": self.skipped[:8]}


def realized_bytes(module: Any) -> dict[str, int]:
    packed = int(module.packed.numel() * module.packed.element_size())
    scale = int(module.scale.numel() * module.scale.element_size())
    bias = 0 if module.bias is None else int(module.bias.numel() * module.bias.element_size())
    return {"packed_bytes": packed, "scale_bytes": scale, "zero_bytes": 0, "bias_bytes": bias,
            "total_bytes": packed + scale + bias}


def set_dequant_mode(model: Any, mode: str) -> int:
    if str(mode) not in DEQUANT_MODES:
        raise ValueError("未知 dequant 模式 %r；可用：%s" % (mode, list(DEQUANT_MODES)))
    n = 0
    for module in model.modules():
        if isinstance(module, QuantLinear):
            module.dequant_mode = str(mode)
            n += 1
    return n


def reset_dequant_counters(model: Any) -> int:
    n = 0
    for module in model.modules():
        if isinstance(module, QuantLinear):
            module._counters = {"separate_calls": 0, "fused_calls": 0, "fallbacks": {}}
            n += 1
    return n


def dequant_activity(model: Any) -> dict[str, Any]:
    """Dispatch counts that really happened (fused vs separate, with fallback reasons)."""
    modes: dict[str, int] = {}
    sep = fus = n = 0
    fallbacks: dict[str, int] = {}
    for module in model.modules():
        if not isinstance(module, QuantLinear):
            continue
        n += 1
        modes[module.dequant_mode] = modes.get(module.dequant_mode, 0) + 1
        sep += int(module._counters["separate_calls"])
        fus += int(module._counters["fused_calls"])
        for reason, count in module._counters["fallbacks"].items():
            fallbacks[reason] = fallbacks.get(reason, 0) + int(count)
    return {"n_quant_linear": n, "modes": modes, "separate_calls": sep, "fused_calls": fus, "fallbacks": fallbacks}


def quantize_model(model: Any, spec: SchemeSpec, *, verbose: bool = False, layers: Any = None,
                   names: Any = None) -> tuple[Any, QuantizeReport]:
    """Replace the ``nn.Linear`` modules selected by ``spec.targets`` with ``QuantLinear`` in place.
    Linears that no rule classifies stay as they are and are listed in ``report.skipped``."""
    report = QuantizeReport(spec=spec.to_dict())
    if not spec.enabled:
        return model, report
    layer_filter = None if layers is None else {int(x) for x in layers}
    name_filter = None if names is None else set(names)
    report.spec["layers"] = None if layer_filter is None else sorted(layer_filter)
    report.spec["names"] = None if name_filter is None else sorted(name_filter)
    candidates = [n for n, m in model.named_modules() if n and isinstance(m, nn.Linear)]
    for module_name in candidates:
        module = model.get_submodule(module_name)
        if not isinstance(module, nn.Linear):
            continue
        target = classify_linear(module_name)
        if target is None:
            report.skipped.append(module_name)
            continue
        if target not in spec.targets:
            report.skipped.append("%s (target=%s 未在 spec.targets 内)" % (module_name, target))
            continue
        if target == "lm_head" and spec.keep_lm_head_fp16:
            report.skipped.append("%s (keep_lm_head_fp16=True)" % module_name)
            continue
        if name_filter is not None and module_name not in name_filter:
            report.skipped.append("%s (不在 names= 白名单内)" % module_name)
            continue
        if layer_filter is not None and _layer_index(module_name) not in layer_filter:
            report.skipped.append("%s (layer 不在 layers= 内)" % module_name)
            continue
        parent_name, _, leaf = module_name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        ql = QuantLinear(module, spec, name=module_name)
        setattr(parent, leaf, ql)
        report.replaced[target] = report.replaced.get(target, 0) + 1
        bucket = report.realized_by_target.setdefault(target, {})
        for key, value in realized_bytes(ql).items():
            bucket[key] = bucket.get(key, 0) + int(value)
        bucket["n_linear"] = bucket.get("n_linear", 0) + 1
        bucket["n_params"] = bucket.get("n_params", 0) + ql.out_features * ql.in_features
        bucket["n_params_padded"] = bucket.get("n_params_padded", 0) + ql.out_features * ql.padded_in
        if verbose:
            print("  quantized %s" % module_name)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    padded = sum(v["n_params_padded"] for v in report.realized_by_target.values())
    unpadded = sum(v["n_params"] for v in report.realized_by_target.values())
    report.padding = {"n_params_padded": padded, "n_params_unpadded": unpadded, "inflation_pct": 0.0}
    return model, report
