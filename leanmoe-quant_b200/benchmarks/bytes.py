"""Per-token byte budgets of the decode step: ``[W]`` (weights streamed) and ``[T] = [W] + KV``
(reference: benchmarks/bytes.py:182-381, extended with an int8-KV term: the reference still books
the KV cache as fp16 after its INT8 read path landed).

Everything is integer arithmetic on the architecture constants; nothing here touches a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class ModelSpec:
    layers: int = 16
    hidden: int = 2048
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    head_dim: int = 128
    num_experts: int = 64
    top_k: int = 8
    expert_ffn_dim: int = 1024
    vocab: int = 50304

    @classmethod
    def from_config(cls, cfg: Any) -> "ModelSpec":
        return cls(layers=cfg.num_hidden_layers, hidden=cfg.hidden_size, num_attention_heads=cfg.num_attention_heads,
                   num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.hidden_size // cfg.num_attention_heads,
                   num_experts=cfg.num_experts, top_k=cfg.num_experts_per_tok, expert_ffn_dim=cfg.intermediate_size,
                   vocab=cfg.vocab_size)


@dataclass(frozen=True)
class QuantSpec:
    bits: int | None = None  # None = fp16 weights
    group_size: int = 128
    scale_dtype_bytes: int = 2
    targets: tuple[str, ...] = ("attention", "experts")
    keep_lm_head_fp16: bool = True

    @property
    def enabled(self) -> bool:
        return self.bits is not None


CANONICAL_QUANT = QuantSpec(bits=8, group_size=128, targets=("attention", "experts", "lm_head"), keep_lm_head_fp16=False)


def _matrix_bytes(rows: int, in_features: int, quant: QuantSpec, quantised: bool, dtype_bytes: int) -> int:
    if not quantised:
        return rows * in_features * dtype_bytes
    groups = -(-in_features // quant.group_size)
    return rows * in_features * int(quant.bits) // 8 + rows * groups * quant.scale_dtype_bytes


def weight_budget(spec: ModelSpec, quant: QuantSpec | None = None, dtype_bytes: int = 2) -> dict[str, Any]:
    """``[W]``: bytes of weights one decoded token streams (only the top-k experts of each layer)."""
    quant = quant or QuantSpec()

    def q(target: str) -> bool:
        if not quant.enabled or target not in quant.targets:
            return False
        return not (target == "lm_head" and quant.keep_lm_head_fp16)

    a = spec.num_attention_heads * spec.head_dim
    kv = spec.num_key_value_heads * spec.head_dim
    items = []
    attn = spec.layers * (_matrix_bytes(a, spec.hidden, quant, q("attention"), dtype_bytes)
                          + 2 * _matrix_bytes(kv, spec.hidden, quant, q("attention"), dtype_bytes)
                          + _matrix_bytes(spec.hidden, a, quant, q("attention"), dtype_bytes))
    items.append({"name": "attention", "bytes": attn, "formula": "layers x (q + k + v + o)"})
    router = spec.layers * _matrix_bytes(spec.num_experts, spec.hidden, quant, q("router"), dtype_bytes)
    items.append({"name": "router", "bytes": router, "formula": "layers x experts x hidden"})
    experts = spec.layers * spec.top_k * (_matrix_bytes(2 * spec.expert_ffn_dim, spec.hidden, quant, q("experts"), dtype_bytes)
                                          + _matrix_bytes(spec.hidden, spec.expert_ffn_dim, quant, q("experts"), dtype_bytes))
    items.append({"name": "experts(top-k)", "bytes": experts, "formula": "layers x top_k x (gate_up + down)"})
    lm_head = _matrix_bytes(spec.vocab, spec.hidden, quant, q("lm_head"), dtype_bytes)
    items.append({"name": "lm_head", "bytes": lm_head, "formula": "vocab x hidden"})
    return {"total_bytes": sum(i["bytes"] for i in items), "items": items}


def kv_budget(spec: ModelSpec, filled: int, kv_int8: bool = False, dtype_bytes: int = 2) -> dict[str, Any]:
    """KV bytes read by one decode step that attends to ``filled`` positions.  int8 mirror: D code
    bytes + one fp16 scale per (layer, K/V, head, position)."""
    per_pos = spec.layers * 2 * spec.num_key_value_heads * ((spec.head_dim + 2) if kv_int8 else spec.head_dim * dtype_bytes)
    return {"total_bytes": per_pos * int(filled), "bytes_per_position": per_pos, "filled": int(filled), "kv_int8": bool(kv_int8)}


def byte_budget(spec: ModelSpec, filled: int, quant: QuantSpec | None = None, kv_int8: bool = False) -> dict[str, Any]:
    """``[T] = [W] + KV`` for one step."""
    w = weight_budget(spec, quant)
    kv = kv_budget(spec, filled, kv_int8)
    return {"W": w["total_bytes"], "KV": kv["total_bytes"], "T": w["total_bytes"] + kv["total_bytes"],
            "weights": w, "kv": kv}


def floor_ms(total_bytes: int, bandwidth_gbs: float) -> float:
    """Time to stream ``total_bytes`` at ``bandwidth_gbs`` (GB/s, 1e9 bytes) in milliseconds."""
    return total_bytes / (bandwidth_gbs * 1e9) * 1e3


def attainment(total_bytes: int, measured_ms: float, bandwidth_gbs: float) -> float:
    """Fraction of the byte floor reached by a measured step time."""
    return floor_ms(total_bytes, bandwidth_gbs) / measured_ms
