"""W8 linear layers and the in-place model pass that installs them (the interface of the reference's
src/lemoq/quant/linear.py: ``SchemeSpec`` :139, ``classify_linear`` :236, ``QuantLinear`` :262, ``quantize_model`` :589).

A :class:`QuantLinear` keeps int8 codes (``packed``) and fp16 group scales (``scale``) as buffers.  A call is served
in one of two ways and counted: ``fused`` - a single fp16 CUDA token goes through the W8 GEMV kernel; ``separate`` -
anything else (prefill, several tokens, another dtype) rebuilds the floating weight and calls ``F.linear``.  Each reason
for leaving the fused way is counted by name.  Only the canonical scheme exists here: ``w8a16``, symmetric, round to
nearest.
"""

from __future__ import annotations

import re
from collections import Counter
from dataclasses import asdict, dataclass, field
from typing import Any, Iterator

import torch
import torch.nn.functional as F
from torch import nn

DEQUANT_MODES = ("separate", "fused")
_SCHEMES = {"w8a16": (8, None), "fp16": (None, None)}  # name -> (weight bits, activation bits)
_ALL_TARGETS = ("attention", "experts", "router")


def parse_scheme(name: str) -> tuple[int | None, int | None]:
    try:
        return _SCHEMES[name]
    except KeyError:
        raise NotImplementedError("scheme %r is not built on this path (canonical decode is w8a16); have %s"
                                  % (name, sorted(_SCHEMES))) from None


def _known_mode(mode: Any) -> str:
    if str(mode) not in DEQUANT_MODES:
        raise ValueError("未知 dequant 模式 %r (unknown dequant mode); have %s" % (mode, list(DEQUANT_MODES)))
    return str(mode)


@dataclass
class SchemeSpec:
    """What to quantise and how.  ``targets`` are classes of linears (see ``TARGET_RULES``)."""

    name: str = "w8a16"
    weight_bits: int | None = 8
    act_bits: int | None = None
    group_size: int = 128
    targets: tuple[str, ...] = _ALL_TARGETS
    keep_lm_head_fp16: bool = True
    symmetric: bool = True
    scheme: str = "rtn"
    dequant: str = "separate"

    def __post_init__(self) -> None:
        self.dequant = _known_mode(self.dequant)

    @classmethod
    def from_flags(cls, name: str, group_size: int, *, targets: tuple[str, ...] | None = None,
                   keep_lm_head_fp16: bool = True, dequant: str = "separate") -> "SchemeSpec":
        weight_bits, act_bits = parse_scheme(name)
        return cls(name, weight_bits, act_bits, group_size, targets or _ALL_TARGETS, keep_lm_head_fp16, dequant=dequant)

    @property
    def enabled(self) -> bool:
        return self.weight_bits is not None

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d["targets"] = list(self.targets)
        d["scheme"], d["rtn_scheme"] = d.pop("name"), d.pop("scheme")
        d["activation_quantization"] = "none"
        return d


# A linear's class follows from its dotted module name; the first rule that matches wins.
TARGET_RULES: tuple[tuple[str, str], ...] = (
    (r"^lm_head$", "lm_head"),
    (r"\.self_attn\.", "attention"),
    (r"\.experts\.\d+\.", "experts"),
    (r"\.mlp\.gate$", "router"),
    (r"\.shared_expert", "shared"),
)
_COMPILED_RULES = tuple((re.compile(pattern), target) for pattern, target in TARGET_RULES)
_LAYER_NUMBER = re.compile(r"\.layers\.(\d+)\.")


def classify_linear(module_name: str) -> str | None:
    return next((target for pattern, target in _COMPILED_RULES if pattern.search(module_name)), None)


def _layer_index(module_name: str) -> int | None:
    found = _LAYER_NUMBER.search(module_name)
    return None if found is None else int(found[1])


def _fresh_counters() -> dict[str, Any]:
    return {"separate_calls": 0, "fused_calls": 0, "fallbacks": {}}


class QuantLinear(nn.Module):
    """Stands in for an ``nn.Linear`` (with or without bias); the weight exists only as int8 codes + group scales."""

    def __init__(self, linear: Any, spec: SchemeSpec, *, name: str = "") -> None:
        from lemoq.quant.rtn import quantize_w8

        super().__init__()
        if spec.weight_bits is None:
            raise ValueError("SchemeSpec.weight_bits 为 None: a spec without weight bits builds no QuantLinear")
        if (int(spec.weight_bits), bool(spec.symmetric), spec.scheme) != (8, True, "rtn"):
            raise NotImplementedError("QuantLinear: only symmetric 8-bit RTN is built (got bits=%r symmetric=%r scheme=%r)"
                                      % (spec.weight_bits, spec.symmetric, spec.scheme))
        group = int(spec.group_size or 0)
        width = int(linear.in_features)
        if group <= 0 or width % group:
            raise NotImplementedError("QuantLinear: in_features=%d 不能被 group_size=%d 整除 (no zero padding on this path)"
                                      % (width, group))
        self.spec, self.name = spec, name
        self.in_features, self.out_features = width, int(linear.out_features)
        self.group_size, self.n_groups, self.padded_in = group, width // group, width
        self.weight_bits = 8
        self.dequant_mode = spec.dequant
        self._counters = _fresh_counters()
        codes, scale = quantize_w8(linear.weight.detach(), group)
        bias = None if linear.bias is None else linear.bias.detach().clone()
        for buffer_name, value in (("packed", codes.contiguous()), ("scale", scale.contiguous()), ("zero", None), ("bias", bias)):
            self.register_buffer(buffer_name, value, persistent=True)

    def dequantized_weight(self, dtype: Any = None) -> Any:
        """``(out, in)`` floating weight = codes x fp16 group scale, in fp32 unless ``dtype`` says otherwise."""
        grouped = (self.out_features, self.n_groups, -1)
        weight = (self.packed.float().view(grouped) * self.scale.float().view(grouped)).view(self.out_features, self.in_features)
        return weight if dtype is None else weight.to(dtype)

    @property
    def fused_available(self) -> bool:
        from lemoq.kernels import dequant_gemv

        return dequant_gemv.unavailable_reason() is None

    def _fused_fallback_reason(self, x: Any) -> str | None:
        """Why this call cannot take the GEMV kernel (None: it can).  The first reason in this order is reported."""
        from lemoq.kernels import dequant_gemv

        checks = (
            (self.dequant_mode == "fused", "mode_is_separate"),
            (x.is_cuda, "not_cuda"),
            (x.dtype == torch.float16, "dtype_unsupported(%s)" % str(x.dtype).removeprefix("torch.")),
            (x.shape[-1] == self.in_features, "input_width_mismatch(%d!=%d)" % (int(x.shape[-1]), self.in_features)),
            (x.numel() == self.in_features, "multi_token"),
        )
        for ok, reason in checks:
            if not ok:
                return reason
        missing = dequant_gemv.unavailable_reason()
        return None if missing is None else (missing or "kernel_unavailable")

    def _fused_forward(self, x: Any) -> Any:
        """The kernel's result, or None (with the reason counted) when the call has to take the other way."""
        reason = self._fused_fallback_reason(x)
        if reason is not None:
            reasons = self._counters["fallbacks"]
            reasons[reason] = reasons.get(reason, 0) + 1
            return None
        from lemoq.kernels.dequant_gemv import dequant_gemm_fused

        row = x.reshape(1, self.in_features).contiguous()
        y = dequant_gemm_fused(row, self.packed, self.scale, None, group_size=self.group_size, bits=8, symmetric=True,
                               out_dtype=x.dtype).reshape(*x.shape[:-1], self.out_features)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def forward(self, x: Any) -> Any:
        y = self._fused_forward(x) if self.dequant_mode == "fused" else None
        if y is not None:
            self._counters["fused_calls"] += 1
            return y
        self._counters["separate_calls"] += 1
        bias = None if self.bias is None else self.bias.to(x.dtype)
        return F.linear(x, self.dequantized_weight(dtype=x.dtype), bias)

    def extra_repr(self) -> str:
        return "%d->%d %s group=%d" % (self.in_features, self.out_features, self.spec.name, self.group_size)


def _quant_linears(model: Any) -> Iterator[QuantLinear]:
    return (m for m in model.modules() if isinstance(m, QuantLinear))


def realized_bytes(module: Any) -> dict[str, int]:
    """Bytes the module really holds, by buffer."""
    size = lambda t: 0 if t is None else int(t.numel() * t.element_size())  # noqa: E731
    parts = {"packed_bytes": size(module.packed), "scale_bytes": size(module.scale), "zero_bytes": 0, "bias_bytes": size(module.bias)}
    return {**parts, "total_bytes": sum(parts.values())}


def set_dequant_mode(model: Any, mode: str) -> int:
    mode = _known_mode(mode)
    count = 0
    for count, module in enumerate(_quant_linears(model), 1):
        module.dequant_mode = mode
    return count


def reset_dequant_counters(model: Any) -> int:
    count = 0
    for count, module in enumerate(_quant_linears(model), 1):
        module._counters = _fresh_counters()
    return count


def dequant_activity(model: Any) -> dict[str, Any]:
    """Which way the calls really went, summed over the model's quantised linears."""
    modes: Counter = Counter()
    calls: Counter = Counter()
    reasons: Counter = Counter()
    for module in _quant_linears(model):
        modes[module.dequant_mode] += 1
        calls.update({k: int(module._counters[k]) for k in ("separate_calls", "fused_calls")})
        reasons.update({k: int(v) for k, v in module._counters["fallbacks"].items()})
    return {"n_quant_linear": sum(modes.values()), "modes": dict(modes), "separate_calls": calls["separate_calls"],
            "fused_calls": calls["fused_calls"], "fallbacks": dict(reasons)}


@dataclass
class QuantizeReport:
    """What ``quantize_model`` did: counts and realised bytes per target class, and every linear it left alone."""

    spec: dict[str, Any]
    replaced: dict[str, int] = field(default_factory=dict)
    skipped: list[str] = field(default_factory=list)
    realized_by_target: dict[str, dict[str, int]] = field(default_factory=dict)
    padding: dict[str, Any] = field(default_factory=dict)

    def count(self, target: str, module: QuantLinear) -> None:
        self.replaced[target] = self.replaced.get(target, 0) + 1
        params = module.out_features * module.in_features
        tally = Counter(self.realized_by_target.get(target, {}))
        tally.update({**realized_bytes(module), "n_linear": 1, "n_params": params,
                      "n_params_padded": module.out_features * module.padded_in})
        self.realized_by_target[target] = dict(tally)

    def close(self) -> None:
        total = lambda key: sum(v.get(key, 0) for v in self.realized_by_target.values())  # noqa: E731
        self.padding = {"n_params_padded": total("n_params_padded"), "n_params_unpadded": total("n_params"), "inflation_pct": 0.0}

    def to_dict(self) -> dict[str, Any]:
        return {"spec": self.spec, "replaced_per_target": self.replaced,
                "realized_bytes_total": sum(v["total_bytes"] for v in self.realized_by_target.values()),
                "realized_bytes_by_target": self.realized_by_target, "padding": self.padding,
                "skipped_linear_count": len(self.skipped), "skipped_linear_examples": self.skipped[:8]}


def _why_skipped(name: str, target: str | None, spec: SchemeSpec, only_names: set | None, only_layers: set | None) -> str | None:
    """The note under which a linear is left unquantised, or None when it is to be replaced."""
    if target is None:
        return name  # no rule knows this linear
    if target not in spec.targets:
        return "%s (target=%s 未在 spec.targets 内)" % (name, target)
    if target == "lm_head" and spec.keep_lm_head_fp16:
        return "%s (keep_lm_head_fp16=True)" % name
    if only_names is not None and name not in only_names:
        return "%s (不在 names= 白名单内)" % name
    if only_layers is not None and _layer_index(name) not in only_layers:
        return "%s (layer 不在 layers= 内)" % name
    return None


def quantize_model(model: Any, spec: SchemeSpec, *, verbose: bool = False, layers: Any = None,
                   names: Any = None) -> tuple[Any, QuantizeReport]:
    """Swap, in place, every ``nn.Linear`` whose class is in ``spec.targets`` for a :class:`QuantLinear`.
    ``layers`` / ``names`` narrow the pass to some decoder layers / exact module names.  Linears left alone are listed
    in ``report.skipped`` with the reason."""
    report = QuantizeReport(spec=spec.to_dict())
    if not spec.enabled:
        return model, report
    only_layers = None if layers is None else {int(n) for n in layers}
    only_names = None if names is None else set(names)
    report.spec["layers"] = None if only_layers is None else sorted(only_layers)
    report.spec["names"] = None if only_names is None else sorted(only_names)
    # the list is taken first: the tree changes while it is walked
    for name in [n for n, m in model.named_modules() if n and isinstance(m, nn.Linear)]:
        target = classify_linear(name)
        note = _why_skipped(name, target, spec, only_names, only_layers)
        if note is not None:
            report.skipped.append(note)
            continue
        owner_name, _, attribute = name.rpartition(".")
        owner = model.get_submodule(owner_name) if owner_name else model
        replacement = QuantLinear(getattr(owner, attribute), spec, name=name)
        setattr(owner, attribute, replacement)
        report.count(target, replacement)
        if verbose:
            print("  quantized %s" % name)
    report.close()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return model, report
