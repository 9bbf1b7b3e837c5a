"""Command-line runner for the decode cell (reference: benchmarks/runner.py:1067-1348, 2447-2944).

    python -m benchmarks.runner --ctx 1024 --bit-width w8a16 --attn kernel --moe grouped \
        --dequant fused --execution cudagraph

Keeps the reference's switches and pre-load refusals for this path and its install order
(norms -> MoE blocks (+ expert quantisation) -> QuantLinear -> attention cores -> packed q.k.v ->
warm -> session -> capture -> graph-vs-eager gate -> timing).  There is no checkpoint or network
here: the model is the OLMoE-1B-7B architecture with seeded random-init fp16 weights.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
if _PKG not in sys.path:
    sys.path.insert(0, _PKG)

from benchmarks.bytes import CANONICAL_QUANT, ModelSpec, QuantSpec, byte_budget  # noqa: E402
from benchmarks.cudagraph import (  # noqa: E402
    CudaGraphCaptureError,
    CudaGraphConfig,
    CudaGraphCorrectnessError,
    StaticCacheDecodeSession,
    compare_logits,
    graph_correctness_passed,
    measure_graph_gap,
    normalize_execution,
)

ARCHITECTURES = ("allenai/OLMoE-1B-7B-0924", "olmoe-1b-7b")
GATED_GROUP_SIZE = 128


class Refusal(ValueError):
    """A cell refused before any model is built (the reference refuses before loading 13 GB)."""


def quant_spec_for_cfg(cfg: dict[str, Any]) -> Any:
    """The cell's ``SchemeSpec`` (None for fp16).  Targets are attention + experts, plus lm_head when
    the ``lm_head_w8`` switch is effective; the router is never quantised."""
    from lemoq.kernels.fusion_switches import fusion_enabled
    from lemoq.quant.linear import SchemeSpec

    bit_width = cfg.get("bit_width") or "fp16"
    if bit_width == "fp16":
        return None
    dequant = str(cfg.get("dequant") or "separate")
    dequant = "separate" if dequant == "none" else dequant
    lmhead = fusion_enabled("lm_head_w8") and bit_width == "w8a16"
    return SchemeSpec.from_flags(str(bit_width), int(cfg.get("group_size") or 128),
                                 targets=("attention", "experts", "lm_head") if lmhead else ("attention", "experts"),
                                 keep_lm_head_fp16=not lmhead, dequant=dequant)


def fused_unavailable_reason() -> str | None:
    try:
        from lemoq.kernels.dequant_gemv import unavailable_reason
    except Exception as exc:  # noqa: BLE001
        return "kernel 模块 import 失败（%s）" % type(exc).__name__
    return unavailable_reason()


def check_refusals(*, ctx: int, batch: int, execution: str, attn: str | None, moe: str, bit_width: str, dequant: str,
                   group_size: int, rmsnorm: str, max_new_tokens: int, timed: int) -> None:
    """Every rule raises ``Refusal`` with a reason; nothing is silently changed."""
    normalize_execution(execution)
    if not (2 <= ctx <= 4096):
        raise Refusal("ctx=%d outside [2, 4096] (model limit)" % ctx)
    if batch != 1:
        raise Refusal("batch=%d: the decode kernels are batch-1" % batch)
    if attn == "kernel" and execution != "cudagraph":
        raise Refusal("--attn kernel needs --execution cudagraph (eager x kernel is not a recorded cell)")
    quantised = bit_width != "fp16"
    if bit_width in ("w8a8", "w4a16"):
        raise Refusal("%s is not built on this path: only fp16 and the canonical w8a16 are" % bit_width)
    if quantised and moe in ("gather", "static"):
        raise Refusal("quantised x gather does not exist: quantisation attaches to the grouped fused tensors")
    if quantised and moe == "hf":
        raise Refusal("quantised x hf MoE cannot be captured")
    if dequant == "fused":
        if not quantised:
            raise Refusal("--dequant fused needs a quantised --bit-width")
        reason = fused_unavailable_reason()
        if reason is not None:
            raise Refusal("--dequant fused unavailable: %s" % reason)
    if quantised and (group_size <= 0 or group_size % 2 != 0):
        raise Refusal("group_size=%d must be a positive even number" % group_size)
    if quantised and group_size != GATED_GROUP_SIZE:
        raise Refusal("group_size=%d has no measured accuracy gate (only %d)" % (group_size, GATED_GROUP_SIZE))
    if rmsnorm == "fused":
        from lemoq.kernels.rmsnorm import unavailable_reason as norm_reason

        r = norm_reason()
        if r is not None:
            raise Refusal("--rmsnorm fused unavailable: %s" % r)
    if execution == "cudagraph":
        CudaGraphConfig(ctx=ctx, max_new_tokens=max_new_tokens, batch=batch).validate_timing(timed)


def build_model(*, layers: int | None = None, seed: int = 0, device: str = "cuda", config: Any = None) -> Any:
    """OLMoE-1B-7B architecture, fp16, seeded ``N(0, 0.02)`` weights generated on ``device``."""
    import torch

    from lemoq.model import OlmoeConfig, OlmoeForCausalLM, init_random_

    cfg = config or OlmoeConfig()
    if layers is not None:
        cfg.num_hidden_layers = int(layers)
    with torch.device(device):
        model = OlmoeForCausalLM(cfg).to(torch.float16)
    return init_random_(model, seed=seed).eval()


def install_replacements(model: Any, *, attn: str | None, moe: str, quant_cfg: dict[str, Any] | None, rmsnorm: str,
                         ctx: int, max_new_tokens: int, device: str = "cuda", prequantized: dict[int, Any] | None = None) -> dict[str, Any]:
    """The reference's install order, all before capture.  ``prequantized`` (layer -> ``QuantFusedExperts``, e.g. from
    ``lemoq.quant.expert_calibration.load_bundle``) supplies the experts ready-made instead of quantising them here."""
    import torch

    from lemoq.kernels.attn_decode import replace_attention_cores, warm as warm_attn
    from lemoq.kernels.moe_static import replace_moe_blocks
    from lemoq.kernels.packed_qkv import install_packed_qkv, packed_qkv_applicable, packed_qkv_enabled
    from lemoq.kernels.rmsnorm import replace_rms_norms
    from lemoq.quant.linear import quantize_model

    info: dict[str, Any] = {}
    info["rmsnorm_replaced"] = replace_rms_norms(model, rmsnorm)
    qspec = quant_spec_for_cfg(quant_cfg) if quant_cfg else None
    if moe != "hf":
        impl = "gather" if moe in ("static", "gather") else "grouped"
        if prequantized is not None:
            info["moe_replaced"] = replace_moe_blocks(model, impl=impl, prequantized=prequantized)
            info["experts_from_bundle"] = True
        else:
            info["moe_replaced"] = replace_moe_blocks(model, impl=impl, quant=qspec)
    if qspec is not None:
        _, report = quantize_model(model, qspec)
        info["quantize_report"] = report.to_dict()
    if attn == "kernel":
        info["attn_replaced"] = replace_attention_cores(model, backend="cuda")
        if packed_qkv_enabled() and packed_qkv_applicable(attn, qspec is not None):
            info["packed_qkv_modules"] = install_packed_qkv(model)
        cfg = model.config
        info["attn_warm"] = warm_attn(heads=cfg.num_attention_heads, head_dim=cfg.head_dim,
                                      kv_len=ctx + max_new_tokens, filled=ctx + max_new_tokens,
                                      dtype=torch.float16, device=device)
    torch.cuda.synchronize()
    return info


def graph_correctness(session: Any, steps: int) -> dict[str, Any]:
    """Graph replay vs the same path run eagerly from the same prefilled state."""
    session.reset()
    seed = session.seed_token_id
    eager_logits, eager_tokens = [], []
    for _ in range(steps):
        eager_logits.append(session.decode_eager().float().cpu().clone())
        eager_tokens.append(session.current_token_id)
    session.reset()
    graph_logits, graph_tokens = [], []
    seed_graph = session.seed_token_id
    for _ in range(steps):
        session.replay(synchronize=True)
        graph_logits.append(session.logits_cpu().float())
        graph_tokens.append(session.current_token_id)
    report = compare_logits(eager_logits, graph_logits)
    report.update(seed_token_match=seed == seed_graph, token_sequence_match=eager_tokens == graph_tokens,
                  steps=steps, tokens=graph_tokens)
    report["passed"] = graph_correctness_passed(report)
    return report


def run_cudagraph(*, ctx: int, max_new_tokens: int = 32, warmup: int = 5, timed: int = 20, attn: str | None = "kernel",
                  moe: str = "grouped", quant_cfg: dict[str, Any] | None = None, rmsnorm: str = "fused",
                  layers: int | None = None, seed: int = 0, device: str = "cuda", engine: str = "auto",
                  bandwidth_gbs: float | None = None, model: Any = None) -> dict[str, Any]:
    import torch

    from lemoq.kernels.fusion_switches import fusion_enabled, fusion_payload_fields

    if model is None:
        model = build_model(layers=layers, seed=seed, device=device)
    info = install_replacements(model, attn=attn, moe=moe, quant_cfg=quant_cfg, rmsnorm=rmsnorm, ctx=ctx,
                                max_new_tokens=max_new_tokens, device=device)
    ids = torch.full((1, ctx), 1, dtype=torch.long, device=device)
    try:
        session = StaticCacheDecodeSession(model, ids, ctx=ctx, max_new_tokens=max_new_tokens, device=device, engine=engine)
    except Exception as exc:  # noqa: BLE001
        raise CudaGraphCaptureError("prefill", exc) from exc
    session.capture(warmup=warmup)
    correctness = graph_correctness(session, max_new_tokens)
    if not correctness["passed"]:
        raise CudaGraphCorrectnessError(correctness)
    timing = measure_graph_gap(session, warmup=warmup, timed=timed)
    spec = ModelSpec.from_config(model.config)
    quant = None
    if quant_cfg and (quant_cfg.get("bit_width") or "fp16") != "fp16":
        lm = fusion_enabled("lm_head_w8")
        quant = CANONICAL_QUANT if lm else QuantSpec(bits=8, group_size=int(quant_cfg.get("group_size") or 128))
    budget = byte_budget(spec, ctx + timed // 2 + 1, quant, kv_int8=fusion_enabled("kv_int8") and attn == "kernel")
    payload = {"status": "measured", "config": {"ctx": ctx, "attn": attn, "moe": moe, "rmsnorm": rmsnorm,
                                                "execution": "cudagraph", **(quant_cfg or {}), **fusion_payload_fields(),
                                                "layers": model.config.num_hidden_layers, "weights": "random-init seed %d" % seed},
               "install": {k: v for k, v in info.items() if k != "quantize_report"},
               "capture": session.capture_info, "correctness": correctness, "timing": timing,
               "bytes": {"W": budget["W"], "KV": budget["KV"], "T": budget["T"]},
               "ms_per_token": timing["wall_p50_ms"], "tok_per_s": 1000.0 / timing["wall_p50_ms"]}
    if bandwidth_gbs:
        floor = budget["T"] / (bandwidth_gbs * 1e9) * 1e3
        payload["floor_ms"] = floor
        payload["floor_fraction_wall"] = floor / timing["wall_p50_ms"]
        payload["floor_fraction_gpu"] = floor / timing["gpu_busy_ms"]
    session.close()
    return payload


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--exp", default="canonical-decode")
    ap.add_argument("--model", default="allenai/OLMoE-1B-7B-0924")
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--timed", type=int, default=20)
    ap.add_argument("--dtype", default="float16")
    ap.add_argument("--execution", default="cudagraph", help="execution arm: eager or cudagraph")
    ap.add_argument("--moe", default="grouped", choices=["hf", "static", "gather", "grouped"])
    ap.add_argument("--static-moe", action="store_true", help="alias of --moe static")
    ap.add_argument("--attn", default="kernel", choices=["sdpa", "eager", "flash_attention_2", "kernel"])
    ap.add_argument("--bit-width", default="w8a16", choices=["fp16", "w8a16", "w8a8", "w4a16"])
    ap.add_argument("--dequant", default="fused", choices=["none", "separate", "fused"])
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--rmsnorm", default="fused", choices=["fused", "hf"])
    ap.add_argument("--results-dir", default="results")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (smoke runs)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--engine", default="auto", choices=["auto", "step", "ops"])
    ap.add_argument("--bandwidth-gbs", type=float, default=None, help="measured HBM bandwidth for the byte floor")
    args = ap.parse_args(argv)

    if args.model not in ARCHITECTURES:
        print(json.dumps({"status": "refused", "reason": "unknown model %r; built: %s (random-init)" % (args.model, ARCHITECTURES)}))
        return 2
    if args.dtype != "float16":
        print(json.dumps({"status": "refused", "reason": "dtype=float16 only"}))
        return 2
    moe = "static" if args.static_moe else args.moe
    try:
        check_refusals(ctx=args.ctx, batch=args.batch, execution=args.execution, attn=args.attn, moe=moe,
                       bit_width=args.bit_width, dequant=args.dequant, group_size=args.group_size, rmsnorm=args.rmsnorm,
                       max_new_tokens=args.max_new_tokens, timed=args.timed)
    except (Refusal, ValueError) as exc:
        print(json.dumps({"status": "refused", "reason": str(exc)}))
        return 2
    cell = "%s__bit_width=%s__dequant=%s__attn=%s__moe=%s__ctx=%d" % (args.exp, args.bit_width, args.dequant, args.attn, moe, args.ctx)
    if args.dry_run:
        print(json.dumps({"status": "dry-run", "cell": cell}))
        return 0
    if args.execution != "cudagraph":
        print(json.dumps({"status": "refused", "reason": "only the cudagraph arm is built"}))
        return 2
    out_dir = os.path.join(args.results_dir, cell)
    out_file = os.path.join(out_dir, "result.json")
    if os.path.exists(out_file) and not args.force:
        print(json.dumps({"status": "done", "cell": cell, "result": out_file}))
        return 0
    quant_cfg = None if args.bit_width == "fp16" else {"bit_width": args.bit_width, "dequant": args.dequant, "group_size": args.group_size}
    try:
        payload = run_cudagraph(ctx=args.ctx, max_new_tokens=args.max_new_tokens, warmup=args.warmup, timed=args.timed,
                                attn=args.attn, moe=moe, quant_cfg=quant_cfg, rmsnorm=args.rmsnorm, layers=args.layers,
                                seed=args.seed, engine=args.engine, bandwidth_gbs=args.bandwidth_gbs)
    except CudaGraphCorrectnessError as exc:
        payload = {"status": "failed", "stage": exc.stage, "report": exc.report, "ms_per_token": None}
    except CudaGraphCaptureError as exc:
        payload = {"status": "blocked", "stage": exc.stage, "error": str(exc)[:1000], "ms_per_token": None}
    payload["cell"] = cell
    os.makedirs(out_dir, exist_ok=True)
    with open(out_file, "w") as fh:
        json.dump(payload, fh, indent=1, default=str)
    print(json.dumps({k: payload.get(k) for k in ("status", "cell", "ms_per_token", "tok_per_s", "floor_fraction_gpu")}))
    return 0 if payload.get("status") == "measured" else 1


if __name__ == "__main__":
    raise SystemExit(main())
