"""Isolated, L2-flushed microbenchmarks of the decode kernels (reference method:
tools/ncu_evidence.py:785-870 and tools/bench_grouped_gemm_quant.py:58-177).

    python leanmoe-quant_b200/benchmarks/bench_kernels.py [--subject moe|dense|attn|all] [--tokens 1,4,16]
                                                          [--iters 20] [--bandwidth-gbs 6552]

Every timed call is one launch (or the two launches of the grouped MoE layer) between two CUDA events on
the current stream, preceded by a 256 MB memset that evicts L2; the median is reported together with
the empty event-pair floor, and GB/s = analytic bytes / (time - floor) as well as / time.

Subjects (benchmark configuration 4 and the per-kernel evidence rows):
  moe    grouped expert GEMV, 64 experts top-8, gate/up [64, 2x1024, 2048], down [64, 2048, 1024]:
         int8 g128 weights with fp16 scales |N(0,1)|*0.01 and the fp16-weight variant, 1/4/16 tokens
  dense  W8 dequant GEMV at the q.k.v (6144x2048), o_proj (2048x2048) and lm_head (50304x2048) shapes
  attn   split-KV decode attention over the int8 mirror and the fp16 cache at ctx 1024 and 4096
One JSON object per line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _PKG not in sys.path:
    sys.path.insert(0, _PKG)

import torch  # noqa: E402

from lemoq import _cabi  # noqa: E402

DEV = "cuda"


class Timer:
    def __init__(self, iters: int) -> None:
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
        floor = []
        for _ in range(20):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            b.record()
            b.synchronize()
            floor.append(a.elapsed_time(b) * 1e3)
        self.floor_us = statistics.median(floor)

    def cold(self, fn, setup=None) -> float:
        """Median microseconds of ``fn()`` over L2-flushed single calls."""
        out = []
        for i in range(self.iters + 3):
            if setup is not None and not (getattr(self, "warm", False) and i > 0):
                setup(i)
            if not getattr(self, "warm", False):
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            if i >= 3:
                out.append(a.elapsed_time(b) * 1e3)
        return statistics.median(out)


def report(name: str, nbytes: int, us: float, floor_us: float, peak: float, **extra) -> None:
    gbs = nbytes / (us * 1e-6) / 1e9
    gbs_net = nbytes / (max(us - floor_us, 1e-3) * 1e-6) / 1e9
    print(json.dumps({"subject": name, "bytes": nbytes, "us_cold": round(us, 2), "event_floor_us": round(floor_us, 2),
                      "gbs": round(gbs, 1), "gbs_minus_floor": round(gbs_net, 1), "frac_of_peak": round(gbs / peak, 4),
                      "frac_minus_floor": round(gbs_net / peak, 4), "peak_gbs": peak, **extra}), flush=True)


def bench_moe(timer: Timer, tokens_list, peak: float) -> None:
    from lemoq.kernels.moe_grouped_quant import QuantFusedExperts

    e, f, h, k = 64, 1024, 2048, 8
    stream = _cabi.current_stream()
    gens = [torch.Generator(device=DEV).manual_seed(s) for s in range(4)]
    gu_c = torch.randint(-127, 128, (e, 2 * f, h), generator=gens[0], dtype=torch.int8, device=DEV)
    dn_c = torch.randint(-127, 128, (e, h, f), generator=gens[1], dtype=torch.int8, device=DEV)
    gu_s = (torch.randn(e, 2 * f, h // 128, generator=gens[2], device=DEV).abs() * 0.01).half()
    dn_s = (torch.randn(e, h, f // 128, generator=gens[3], device=DEV).abs() * 0.01).half()
    q = QuantFusedExperts(gu_c, gu_s, dn_c, dn_s, 8, 128)
    per_expert_w8 = 2 * f * h + 2 * f * (h // 128) * 2 + h * f + h * (f // 128) * 2
    for t in tokens_list:
        g = torch.Generator(device=DEV).manual_seed(10 + t)
        x = torch.randn(t, h, generator=g, device=DEV).half()
        act = torch.empty((t, k, f), dtype=torch.float16, device=DEV)
        out = torch.empty((t, h), dtype=torch.float16, device=DEV)
        state = {}

        def setup(i):
            logits = torch.randn(t, e, generator=g, device=DEV)
            w, ids = torch.topk(torch.softmax(logits, dim=-1), k, dim=-1)
            state["ids"], state["w"] = ids.contiguous(), w.half().contiguous()

        def both():
            _cabi.call("lemoq_moe_grouped_w8", _cabi.ptr(x), _cabi.ptr(gu_c), _cabi.ptr(gu_s), _cabi.ptr(dn_c), _cabi.ptr(dn_s),
                       _cabi.ptr(state["ids"]), _cabi.ptr(state["w"]), t, k, e, h, f, 128, _cabi.ptr(act), _cabi.ptr(out), None, stream)

        def gate_up():
            _cabi.call("lemoq_moe_gate_up_w8", _cabi.ptr(x), _cabi.ptr(gu_c), _cabi.ptr(gu_s), _cabi.ptr(state["ids"]), t, k, e, h, f,
                       128, _cabi.ptr(act), None, stream)

        def down():
            _cabi.call("lemoq_moe_down_w8", _cabi.ptr(act), _cabi.ptr(dn_c), _cabi.ptr(dn_s), _cabi.ptr(state["ids"]),
                       _cabi.ptr(state["w"]), t, k, e, h, f, 128, _cabi.ptr(out), None, stream)

        setup(0)
        distinct = int(torch.unique(state["ids"]).numel())
        us = timer.cold(both, setup)
        report("moe_grouped_w8 (gate_up+down)", distinct * per_expert_w8 + t * h * 2 * 2, us, timer.floor_us, peak, tokens=t,
               distinct_experts=distinct, note="bytes count each distinct expert once")
        if t > 1:
            # the many-token form: pairs sorted by expert, weights-stationary kernels (each distinct expert read once)
            from lemoq.kernels.batched_w8 import expert_segments, w8_experts_tokens

            def sorted_pairs():
                flat = state["ids"].reshape(-1)
                order = torch.argsort(flat, stable=True)
                state["pair_x"] = x[torch.div(order, k, rounding_mode="floor")].contiguous()
                state["pair_e"] = flat[order].contiguous()
                state["seg"] = expert_segments(state["pair_e"], e)

            def setup_pairs(i):
                setup(i)
                sorted_pairs()

            def many():
                w8_experts_tokens(state["pair_x"], state["pair_e"], gu_c, gu_s, dn_c, dn_s, group_size=128, seg_offsets=state["seg"])

            setup_pairs(0)
            distinct = int(torch.unique(state["ids"]).numel())
            us = timer.cold(many, setup_pairs)
            report("moe_w8 many-token kernels (quantise + gate_up + quantise + down, pairs sorted by expert)",
                   distinct * per_expert_w8 + t * h * 2 * 2, us, timer.floor_us, peak, tokens=t, distinct_experts=distinct,
                   note="bytes count each distinct expert once; the sort, the segment offsets and the routing-weighted combine are outside")
        if t == 1:
            us = timer.cold(gate_up, setup)
            report("moe_gate_up_w8", k * (2 * f * h + 2 * f * (h // 128) * 2) + h * 2 + k * f * 2, us, timer.floor_us, peak, tokens=t)
            us = timer.cold(down, setup)
            report("moe_down_w8", k * (h * f + h * (f // 128) * 2) + k * f * 2 + h * 2, us, timer.floor_us, peak, tokens=t)
    del q
    # fp16-weight variant (one token)
    from lemoq.kernels.moe_grouped import grouped_moe_forward
    from lemoq.kernels.moe_static import FusedExperts

    fused = FusedExperts((torch.randn(e, 2 * f, h, generator=gens[0], device=DEV) * 0.02).half(),
                         (torch.randn(e, h, f, generator=gens[1], device=DEV) * 0.02).half())
    x = torch.randn(h, generator=gens[2], device=DEV).half()
    state = {}

    def setup16(i):
        logits = torch.randn(1, e, generator=gens[3], device=DEV)
        w, ids = torch.topk(torch.softmax(logits, dim=-1), k, dim=-1)
        state["ids"], state["w"] = ids.reshape(-1).contiguous(), w.reshape(-1).half().contiguous()

    act = torch.empty((k, f), dtype=torch.float16, device=DEV)
    out = torch.empty((h,), dtype=torch.float16, device=DEV)

    def both16():
        _cabi.call("lemoq_moe_grouped_fp16", _cabi.ptr(x), _cabi.ptr(fused.gate_up), _cabi.ptr(fused.down), _cabi.ptr(state["ids"]),
                   _cabi.ptr(state["w"]), 1, k, e, h, f, _cabi.ptr(act), _cabi.ptr(out), None, stream)

    us = timer.cold(both16, setup16)
    report("moe_grouped_fp16 (gate_up+down)", k * 3 * f * h * 2 + h * 4, us, timer.floor_us, peak, tokens=1)
    _ = grouped_moe_forward


def bench_dense_tokens(timer: Timer, peak: float) -> None:
    """The weights-stationary dense kernel at the q.k.v and lm_head shapes for 16 and 64 tokens."""
    from lemoq.kernels.batched_w8 import quantise_tokens, w8_rows_tokens

    for name, n in (("qkv 6144x2048", 6144), ("lm_head 50304x2048", 50304)):
        g = torch.Generator(device=DEV).manual_seed(n)
        codes = torch.randint(-127, 128, (n, 2048), generator=g, dtype=torch.int8, device=DEV)
        scale = (torch.randn(n, 16, generator=g, device=DEV).abs() * 0.01).half()
        for t in (16, 64):
            x = torch.randn(t, 2048, generator=g, device=DEV).half()

            def run():
                w8_rows_tokens(quantise_tokens(x), t, codes, scale, group_size=128)

            us = timer.cold(run, lambda i: None)
            report("dense_w8 many-token kernel %s" % name, n * 2048 + n * 16 * 2 + t * 2048 * 2 + t * n * 2, us, timer.floor_us, peak, tokens=t)


def bench_dense(timer: Timer, peak: float) -> None:
    stream = _cabi.current_stream()
    g = torch.Generator(device=DEV).manual_seed(0)
    for name, n, k in (("dense_w8 qkv 6144x2048", 6144, 2048), ("dense_w8 o_proj 2048x2048", 2048, 2048),
                       ("dense_w8 lm_head 50304x2048", 50304, 2048)):
        codes = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8, device=DEV)
        scale = (torch.rand(n, k // 128, generator=g, device=DEV) * 0.01).half()
        x = torch.randn(1, k, generator=g, device=DEV).half()
        y = torch.empty((1, n), dtype=torch.float16, device=DEV)
        us = timer.cold(lambda: _cabi.call("lemoq_dequant_gemv_w8", _cabi.ptr(x), 1, _cabi.ptr(codes), _cabi.ptr(scale), n, k, 128,
                                           _cabi.ptr(y), 0, stream))
        report(name, n * k + n * (k // 128) * 2 + k * 2 + n * 2, us, timer.floor_us, peak)


def bench_attn(timer: Timer, peak: float) -> None:
    stream = _cabi.current_stream()
    g = torch.Generator(device=DEV).manual_seed(1)
    heads, d = 16, 128
    for ctx in (1024, 4096):
        s = ctx + 32
        q = torch.randn(heads, d, generator=g, device=DEV).half()
        k16 = torch.randn(heads, s, d, generator=g, device=DEV).half()
        v16 = torch.randn(heads, s, d, generator=g, device=DEV).half()
        kc = torch.randint(-127, 128, (heads, s, d), generator=g, dtype=torch.int8, device=DEV)
        vc = torch.randint(-127, 128, (heads, s, d), generator=g, dtype=torch.int8, device=DEV)
        ks = (torch.rand(heads, s, generator=g, device=DEV) * 0.02).half()
        vs = (torch.rand(heads, s, generator=g, device=DEV) * 0.02).half()
        out = torch.empty((heads, d), dtype=torch.float16, device=DEV)
        filled = torch.tensor([ctx + 1], dtype=torch.int32, device=DEV)
        for splits in (10, 19, 37):
            ws = torch.zeros(int(_cabi.lib().lemoq_attn_workspace_bytes(heads, d, splits)), dtype=torch.uint8, device=DEV)
            us = timer.cold(lambda: _cabi.call("lemoq_attn_decode_int8", _cabi.ptr(q), _cabi.ptr(kc), _cabi.ptr(ks), _cabi.ptr(vc),
                                               _cabi.ptr(vs), s * d, _cabi.ptr(filled), _cabi.ptr(out), heads, s, d, splits,
                                               d ** -0.5, _cabi.ptr(ws), None, stream))
            report("attn_int8 ctx%d" % ctx, (ctx + 1) * heads * (d + 2) * 2, us, timer.floor_us, peak, splits=splits)
            us = timer.cold(lambda: _cabi.call("lemoq_attn_decode_fp16", _cabi.ptr(q), _cabi.ptr(k16), _cabi.ptr(v16), s * d,
                                               _cabi.ptr(filled), _cabi.ptr(out), heads, s, d, splits, d ** -0.5, _cabi.ptr(ws),
                                               None, stream))
            report("attn_fp16 ctx%d" % ctx, (ctx + 1) * heads * d * 2 * 2, us, timer.floor_us, peak, splits=splits)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--subject", default="all", choices=["moe", "dense", "attn", "all"])
    ap.add_argument("--tokens", default="1,4,16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--bandwidth-gbs", type=float, default=None)
    ap.add_argument("--dot-mode", type=int, default=None, help="lemoq_set_tuning key 0 (0 magic fp32, 1 exact cvt, 2 exact mixed)")
    ap.add_argument("--warm", action="store_true", help="no L2 flush between calls (data served from L2 when it fits)")
    ap.add_argument("--warps", type=int, default=None, help="lemoq_set_tuning key 1: warps per block of the streaming kernels")
    args = ap.parse_args()
    peak = args.bandwidth_gbs
    if peak is None:
        path = os.path.join(os.path.dirname(_PKG), "MEASURED_PEAKS.json")
        peak = float(json.load(open(path))["hbm_gbs"]) if os.path.exists(path) else 6650.0
    _cabi.lib()
    if args.dot_mode is not None:
        _cabi.call("lemoq_set_tuning", 0, args.dot_mode)
    if args.warps is not None:
        _cabi.call("lemoq_set_tuning", 1, args.warps)
    print(json.dumps({"tuning": {"dot_mode": args.dot_mode, "warps": args.warps}}), flush=True)
    timer = Timer(args.iters)
    timer.warm = args.warm
    if args.subject in ("moe", "all"):
        bench_moe(timer, [int(t) for t in args.tokens.split(",")], peak)
    if args.subject in ("dense", "all"):
        bench_dense(timer, peak)
        bench_dense_tokens(timer, peak)
    if args.subject in ("attn", "all"):
        bench_attn(timer, peak)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
