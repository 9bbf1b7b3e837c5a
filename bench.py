"""Benchmark of the hot path: batch-1 greedy decode of the canonical OLMoE cell.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--ctx 1024] [--impl reference]

Workload (benchmark configuration 2): full OLMoE-1B-7B architecture (16 layers, hidden 2048, 64 experts top-8,
expert FFN 1024, vocab 50304), seeded random-init fp16 weights, canonical quantisation W8A16 g128 +
lm_head W8 + per-token INT8 KV, all-ones prompt of ``ctx`` tokens prefilled, then greedy decode.
A "step" is one decoded token = one replay of the captured step graph.

Printed JSON line (rank 0):
  value   tokens/s with everything on the device: the step feeds itself (its pick, the next slot and the next
          length go into its own input scalars), the timed region is K graph replays, device-timed with CUDA events.
  e2e     tokens/s through the public session API with host buffers: ``replay_chained(32)`` copies the first
          step's inputs from pinned host memory (32 B), replays 32 steps and reads the 32 token ids back (8 B each)
          with one synchronisation; ``e2e.per_token_sync`` is the reference's loop (inputs in, replay, synchronise,
          token out, every step).
  roofline  the dominant kernel.  With the whole-step kernel (default) that is the one launch per step:
          the step's algorithmic bytes / the device-timed step against the measured HBM copy bandwidth.
          With chained kernels it is the expert gate/up GEMV timed alone on L2-flushed launches (also
          reported beside the whole-step figure).
  cpu_baseline  the CPU oracle (a port of the reference's torch CPU path) on a bounded sample (one GPU only).
  ctx4096 / config4 / expert_parallel  sub-records: benchmark configuration 3 (ctx 4096, int8 and fp16 KV),
          configuration 4 (isolated L2-flushed kernels) and configuration 5 (64 sequences x ctx 2048, experts
          sharded over the N ranks with NCCL all-to-all; at N = 1 the same decoder without the exchange).

``--impl reference`` times only that CPU implementation (all host threads) on the same configuration.
With ``--gpus N`` (under torchrun) batch-1 decode does not shard: every rank runs an independent
replica ("replicas only"), the reported value is the sum over ranks with the max-over-ranks time; the
``expert_parallel`` sub-record is the one measurement in which the N ranks work on one job.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "leanmoe-quant_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "decode_tokens_per_s_batch1"
UNIT = "tok/s"


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback (6.65 TB/s, earlier measurement on this pool)"}


def workload_config(ctx: int, layers: int, world: int, bytes_first_step: int) -> dict:
    """The ``config`` block both arms print: the workload, nothing about how an arm runs it (``bytes_first_step``: the
    byte model at the first decoded position, so that the text does not depend on how many steps an arm times)."""
    return {"workload": "OLMoE-1B-7B architecture batch-1 greedy decode, W8A16 g128 + lm_head W8 + INT8 KV, "
                        "ctx %d, one decoded token per step (benchmark configuration 2)" % ctx,
            "ctx": ctx, "layers": layers,
            "l2": "inputs larger than L2: %.2f GB streamed per step vs 126 MB L2" % (bytes_first_step / 1e9),
            "parallelism": "replicas only" if world > 1 else "single GPU"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's torch CPU path on synthetic quantised weights
# ----------------------------------------------------------------------------------------------
def synthetic_oracle_weights(spec, seed: int = 0):
    """Quantised weights drawn directly (int8 codes uniform, fp16 scales |N(0,1)|*0.01 scaled down):
    the values do not change the work a step does, and drawing codes avoids minutes of CPU RTN."""
    import torch

    from oracle import lemoq_oracle as ops
    from oracle import olmoe_decode_oracle as glue

    g = torch.Generator().manual_seed(seed)

    def codes(*shape):
        return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)

    def scales(*shape):
        return (torch.rand(shape, generator=g) * 2.0e-4 + 1.0e-4).half()

    h, a, e, f, grp = spec.hidden, spec.attn_dim, spec.experts, spec.ffn, spec.group_size
    ones = torch.ones(h, dtype=torch.float16)
    layers = []
    for _ in range(spec.layers):
        ex = ops.QuantExperts(codes(e, 2 * f, h), scales(e, 2 * f, h // grp), codes(e, h, f), scales(e, h, f // grp), grp)
        layers.append(glue.LayerWeights(ln1=ones, ln2=ones, q_norm=torch.ones(a, dtype=torch.float16),
                                        k_norm=torch.ones(a, dtype=torch.float16),
                                        router=(torch.randn(e, h, generator=g) * 0.02).half(),
                                        qkv_codes=codes(3 * a, h), qkv_scale=scales(3 * a, h // grp),
                                        o_codes=codes(h, a), o_scale=scales(h, a // grp), experts=ex))
    return glue.ModelWeights(spec=spec, embed=(torch.randn(spec.vocab, h, generator=g) * 0.02).half(), layers=layers,
                             final_norm=ones, lm_head_codes=codes(spec.vocab, h), lm_head_scale=scales(spec.vocab, h // grp),
                             quantized=True)


def time_oracle_steps(wq, st, first_token: int, ctx: int, steps: int, warmup: int):
    """Greedy decode on the CPU oracle; returns the list of per-step seconds (timed steps only)."""
    import torch

    from oracle import olmoe_decode_oracle as glue

    tok, times = int(first_token), []
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        lg = glue.decode_step(wq, st, tok, ctx + s, kv_int8=True)
        tok = int(torch.argmax(lg.float()))
        if s >= warmup:
            times.append(time.perf_counter() - t0)
    return times


REFERENCE_MAX_STEPS = 60


def run_reference(args) -> int:
    """The reference arm: the CPU implementation of the decode step on the host cores."""
    import torch

    from oracle import olmoe_decode_oracle as glue

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    spec = glue.OlmoeSpec()
    steps, warmup = max(1, args.steps), max(1, args.warmup)
    # a CPU step takes most of a second: at most 60 of the K steps (and 3 warm-up steps) are run, so that the arm ends
    # within a minute or two whatever K is; the line says how many were timed
    timed, warm = min(steps, REFERENCE_MAX_STEPS), min(warmup, 3)
    wq = synthetic_oracle_weights(spec)
    st = glue.new_state(spec, args.ctx + timed + warm)
    g = torch.Generator().manual_seed(1)
    for i in range(spec.layers):
        st.keys[i][:, :, : args.ctx] = torch.randn(1, spec.heads, args.ctx, spec.head_dim, generator=g).half()
        st.values[i][:, :, : args.ctx] = torch.randn(1, spec.heads, args.ctx, spec.head_dim, generator=g).half()
    glue.build_int8_mirror(st)
    times = time_oracle_steps(wq, st, 1, args.ctx, timed, warm)
    ms = 1000.0 * sum(times) / len(times)
    value = 1000.0 / ms
    sample = "%d decode steps (of --steps %d; %d warm-up) of the 16-layer canonical model at ctx %d (synthetic int8 codes, random fp16 KV)" % (
        timed, steps, warm, args.ctx)
    from benchmarks.bytes import CANONICAL_QUANT, ModelSpec, byte_budget
    from lemoq.model import OlmoeConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    first = byte_budget(ModelSpec.from_config(OlmoeConfig()), args.ctx + 1, CANONICAL_QUANT, kv_int8=True)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "steps_timed": timed, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights/KV, fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": workload_config(args.ctx, spec.layers, world, first["T"]),
        "run": {"weights": "synthetic int8 codes and fp16 scales of the canonical shapes (the work of a step does not depend on the values)",
                "threads": torch.get_num_threads()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))
    return 0


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum of one step_tile_kernel launch, from one ncu capture of
# `python bench.py --steps 4 --warmup 3 --no-cpu-baseline --no-sub-records` (summary under profiles/):
# (ctx, layers) -> bytes.
WHOLE_STEP_DRAM_TRAFFIC = {(1024, 16): 1269527296 + 4218624}


def time_dominant_kernel(model, peaks, iters: int = 20) -> dict:
    """Expert gate/up GEMV (the kernel with the largest byte share of a step) timed alone: one launch
    per event pair on the current stream, a 256 MB L2 flush before every launch."""
    import torch

    from lemoq import _cabi

    cfg = model.config
    ex = model.model.layers[0].mlp._static_experts
    dev = ex.packed_gate_up.device
    k, h, f, e = cfg.num_experts_per_tok, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    x = torch.randn(h, device=dev).half()
    act = torch.empty((k, f), dtype=torch.float16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = _cabi.current_stream(dev)
    times = []
    for i in range(iters + 3):
        ids = (torch.randperm(e, device=dev)[:k]).to(torch.int64)
        layer = model.model.layers[i % cfg.num_hidden_layers].mlp._static_experts
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _cabi.call("lemoq_moe_gate_up_w8", _cabi.ptr(x), _cabi.ptr(layer.packed_gate_up), _cabi.ptr(layer.scale_gate_up),
                   _cabi.ptr(ids), 1, k, e, h, f, int(layer.group_size), _cabi.ptr(act), None, stream)
        end.record()
        end.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(end) * 1e-3)
    # event-pair floor (empty region) so that launch latency is not booked as bandwidth
    floor = []
    for _ in range(10):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        end.record()
        end.synchronize()
        floor.append(start.elapsed_time(end) * 1e-3)
    nbytes = k * (2 * f * h + 2 * f * (h // int(ex.group_size)) * 2) + h * 2 + k * f * 2
    t = statistics.median(times)
    achieved = nbytes / t / 1e9
    return {"bound": "hbm", "kernel": "stream_gate_up_kernel (expert gate/up W8 GEMV + SwiGLU, lemoq_moe_gate_up_w8)", "achieved": achieved,
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
            "bytes_per_launch": nbytes, "us_per_launch": t * 1e6, "event_floor_us": statistics.median(floor) * 1e6,
            "peak_source": peaks["source"], "timing": "CUDA events, isolated launches, 256 MB L2 flush before each"}


def sub_ctx4096(model, peaks, device: str, steps: int = 64) -> dict:
    """Benchmark configuration 3: the same model at ctx 4096, attending to the int8 mirror (whole-step kernel) and,
    for comparison, to the fp16 cache (kv_int8 switched off: chained kernels).  Device-timed self-feeding replays."""
    import torch

    from benchmarks.bytes import CANONICAL_QUANT, ModelSpec, byte_budget
    from benchmarks.cudagraph import StaticCacheDecodeSession

    ctx, horizon = 4096, steps + 8
    spec = ModelSpec.from_config(model.config)
    prompt = torch.full((1, ctx), 1, dtype=torch.long, device=device)
    out = {"ctx": ctx, "steps": steps, "what": "benchmark configuration 3; device-timed, %d self-feeding graph replays after 5 warm-up steps" % steps}
    for name, kv_int8 in (("kv_int8", True), ("kv_fp16", False)):
        old = os.environ.get("LEMOQ_KV_INT8")
        os.environ["LEMOQ_KV_INT8"] = "1" if kv_int8 else "0"
        try:
            session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=horizon, device=device, engine="step")
            session.capture(warmup=3)
        finally:
            if old is None:
                os.environ.pop("LEMOQ_KV_INT8", None)
            else:
                os.environ["LEMOQ_KV_INT8"] = old
        session.reset()
        for _ in range(5):
            session.replay(synchronize=True)
        session._set_step_inputs(skip_mask=session._replay_skip_mask())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(session.stream):
            e0.record(session.stream)
            for _ in range(steps):
                session.graph.replay()
            e1.record(session.stream)
        session.stream.synchronize()
        ms = e0.elapsed_time(e1) / steps
        budget = byte_budget(spec, ctx + 5 + steps // 2 + 1, CANONICAL_QUANT, kv_int8=kv_int8)
        floor = budget["T"] / (peaks["hbm_gbs"] * 1e9) * 1e3
        out[name] = {"ms_per_token": ms, "tok_per_s": 1000.0 / ms, "bytes_per_step": budget["T"], "byte_floor_ms": floor,
                     "floor_fraction": floor / ms, "kernels_per_step": session.capture_info.get("kernels_per_step"),
                     "step_kernel": session.capture_info.get("step_kernel"), "error_flags": session.step_error_flags()}
        session.close()
        del session
        torch.cuda.empty_cache()
    return out


def sub_config4(peaks) -> dict:
    """Benchmark configuration 4 and the per-kernel rows: the isolated, L2-flushed microbenchmarks of
    benchmarks/bench_kernels.py (grouped MoE at 1/4/16 tokens with int8 and fp16 weights, dense W8 rows at the
    q.k.v / o_proj / lm_head shapes for one token and, with the many-token kernel, for 16 and 64, attention at
    ctx 1024 / 4096 for three split counts)."""
    import contextlib
    import io

    from benchmarks import bench_kernels as bk

    buf = io.StringIO()
    timer = bk.Timer(10)
    with contextlib.redirect_stdout(buf):
        bk.bench_moe(timer, [1, 4, 16], peaks["hbm_gbs"])
        bk.bench_dense(timer, peaks["hbm_gbs"])
        bk.bench_dense_tokens(timer, peaks["hbm_gbs"])
        bk.bench_attn(timer, peaks["hbm_gbs"])
    rows = []
    for line in buf.getvalue().splitlines():
        line = line.strip()
        if line.startswith("{"):
            r = json.loads(line)
            rows.append({k: r[k] for k in ("subject", "bytes", "us_cold", "gbs", "frac_of_peak", "frac_minus_floor") if k in r}
                        | {k: r[k] for k in ("tokens", "weights", "ctx", "kv", "splits") if k in r})
    return {"what": "isolated launches, 256 MB L2 flush before each, median of 10, GB/s = analytic bytes / time; "
                    "frac_minus_floor subtracts the empty event-pair time (%.1f us)" % timer.floor_us,
            "peak_gbs": peaks["hbm_gbs"], "rows": rows}


EP_GOLDEN = os.path.join(ROOT, "tests", "golden", "expert_parallel_tokens.json")


def sub_expert_parallel(model, device: str, world: int, rank: int) -> dict:
    """Benchmark configuration 5 on this run's GPUs: 64 sequences x ctx 2048 in lockstep, experts sharded over the
    ranks, static-capacity NCCL all-to-all, the whole step in one CUDA graph.  ``tokens_match_one_gpu`` compares the
    digest of all decoded tokens with the committed digest of the same run on one GPU."""
    from benchmarks import expert_parallel as ep

    rec = ep.measure(model, device=device, world=world, rank=rank, sequences=64, ctx=2048, steps=32, warmup=3,
                     exchange="static", graph=True, split=True)
    rec.pop("tokens")
    want = None
    if os.path.exists(EP_GOLDEN):
        with open(EP_GOLDEN) as fh:
            want = json.load(fh).get("sha256")
    rec["tokens_match_one_gpu"] = (rec["token_digest"] == want) if want else None
    return rec


def run_gpu(args) -> int:
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    device = "cuda:%d" % local_rank

    from benchmarks.bytes import CANONICAL_QUANT, ModelSpec, byte_budget
    from benchmarks.cudagraph import StaticCacheDecodeSession
    from benchmarks.runner import build_model, install_replacements
    from lemoq import _cabi

    _cabi.lib()  # the CUDA library must be there: no fallback
    peaks = measured_peaks()
    steps, warmup, ctx = max(1, args.steps), max(3, args.warmup), args.ctx
    horizon = steps + warmup + 2
    model = build_model(seed=0, device=device, layers=args.layers)
    install_replacements(model, attn="kernel", moe="grouped",
                         quant_cfg={"bit_width": "w8a16", "dequant": "fused", "group_size": 128}, rmsnorm="fused",
                         ctx=ctx, max_new_tokens=horizon, device=device)
    prompt = torch.full((1, ctx), 1, dtype=torch.long, device=device)
    session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=horizon, device=device, engine=args.engine)
    session.capture(warmup=3)
    launches_per_step = int(session.capture_info.get("kernels_per_step") or 0)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    # ---------------- value: device-resident inputs, K replays at advancing positions ----------------
    torch.cuda.synchronize()
    t_prefill = time.perf_counter()
    session.reset()  # the eager prefill of the prompt (context only: it is not part of the metric)
    torch.cuda.synchronize()
    prefill_ms = (time.perf_counter() - t_prefill) * 1e3
    for _ in range(warmup):
        session.replay(synchronize=True)
    start_pos = session.position
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the step feeds itself on the device (its pick, the next slot and the next length go into its own input scalars):
    # the scalars of the first step are set before the clock starts, the timed region is K graph replays
    native = session.capture_info.get("engine") == "step"
    if native:
        session._set_step_inputs(skip_mask=session._replay_skip_mask())
    torch.cuda.synchronize()
    with torch.cuda.stream(session.stream):
        ev0.record(session.stream)
        for i in range(steps):
            if native:
                session.graph.replay()
            else:  # the per-op engine needs its inputs and an attention mask from the host every step
                session.position = start_pos + i
                session.replay(synchronize=False)
        ev1.record(session.stream)
    session.stream.synchronize()
    barrier()
    dev_ms = max_over_ranks(ev0.elapsed_time(ev1)) / steps
    # where the last timed step spent its time: block 0's time stamps at the phase boundaries of the whole-step kernel
    phase_us = None
    stamps = session.step_phase_times_us() if native else None
    if stamps is not None:
        rows = stamps["phases"][1:] if stamps["phases"].shape[0] > 1 else stamps["phases"]  # layer 0 starts cold
        phase_us = {"order": ["q.k.v", "attention", "o_proj", "router", "gate_up", "down"],
                    "per_layer_mean": [round(float(v), 2) for v in rows.mean(0)],
                    "lm_head": round(float(stamps["lm_head"]), 2), "step": round(float(stamps["total"]), 2)}
    # ---------------- e2e: the public session API with host buffers ----------------
    # replay_chained(B): the first step's inputs come from pinned host memory (one 32-byte copy), B replays run with
    # no host work in between, the B token ids come back in one copy to pinned host memory; the host continues from
    # the last token.  B = 32 is the reference's decode horizon (32 greedy steps).
    block = 32
    session.reset()
    for _ in range(warmup):
        session.replay(synchronize=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record(session.stream)
    done = 0
    if native:
        while done < steps:
            n = min(block, steps - done)
            session.replay_chained(n)
            done += n
    else:
        for i in range(steps):
            session.replay(synchronize=True)
    e1.record(session.stream)
    session.stream.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1000.0 / steps
    barrier()
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1) / steps, wall_ms))
    # the reference's loop for comparison: inputs in, replay, synchronize, token out, every single step
    session.reset()
    for _ in range(warmup):
        session.replay(synchronize=True)
    pinned_in = torch.zeros(4, dtype=torch.int64).pin_memory()
    pinned_out = torch.zeros(1, dtype=torch.int64).pin_memory()
    b = session.buffers
    tok, pos = session.current_token_id, session.position
    nsync = min(steps, 100)
    barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(session.stream):
        for i in range(nsync):
            b.pack_step(pinned_in, token=tok, position=pos + i)
            b.packed.copy_(pinned_in, non_blocking=True)
            session.graph.replay()
            picked = session.step_next_token
            if picked is None:
                picked = session.logits.reshape(-1).argmax().reshape(1)
            pinned_out.copy_(picked, non_blocking=True)
            session.stream.synchronize()
            tok = int(pinned_out[0])
    per_token_sync_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0 / nsync)
    barrier()
    clocks = sampler.stop()

    spec = ModelSpec.from_config(model.config)
    budget = byte_budget(spec, ctx + warmup + steps // 2 + 1, CANONICAL_QUANT, kv_int8=True)
    floor_ms = budget["T"] / (peaks["hbm_gbs"] * 1e9) * 1e3
    result = {
        "metric": METRIC, "value": world * 1000.0 / dev_ms, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights/KV, fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": workload_config(ctx, model.config.num_hidden_layers, world, byte_budget(spec, ctx + 1, CANONICAL_QUANT, kv_int8=True)["T"]),
        "run": {"engine": session.capture_info.get("engine"), "step_kernel": session.capture_info.get("step_kernel"),
                "pdl": session.capture_info.get("pdl"), "weights": "random-init N(0,0.02) seed 0, RTN-quantised on the GPU",
                "execution": "one CUDA graph per step", "prefill_ms": round(prefill_ms, 1), "phase_us": phase_us},
        "ms_per_token": dev_ms, "bytes_per_step": budget["T"], "byte_floor_ms": floor_ms,
        "floor_fraction": floor_ms / dev_ms, "floor_fraction_e2e": floor_ms / e2e_ms,
        "e2e": {"value": world * 1000.0 / e2e_ms, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 32.0 / block if native else 32, "d2h_bytes_per_step": 8,
                "api": "StaticCacheDecodeSession.replay_chained(32): 32 B of step inputs in per 32 tokens, 8 B per token out, "
                       "one synchronisation per 32 tokens" if native else "StaticCacheDecodeSession.replay per token",
                "per_token_sync": {"value": world * 1000.0 / per_token_sync_ms, "unit": UNIT, "ms_per_step": per_token_sync_ms,
                                   "h2d_bytes_per_step": 32, "d2h_bytes_per_step": 8,
                                   "what": "the reference's loop: inputs in, replay, synchronise, token out, every step"}},
        "gpu_launches": launches_per_step * (2 * steps + nsync), "kernels_per_step": launches_per_step,
        "step_kernel": session.capture_info.get("step_kernel"), "clocks": clocks,
    }
    if rank == 0:
        isolated = time_dominant_kernel(model, peaks)
        if launches_per_step == 1:
            # The whole step is ONE kernel launch: that kernel is the dominant kernel.  Its average launch
            # duration is the device-timed step of the timed region above (CUDA events on the launching stream).
            achieved = budget["T"] / (dev_ms * 1e-3) / 1e9
            result["roofline"] = {
                "bound": "hbm", "kernel": "step_tile_kernel (whole decode step: 16 x 6 phases + lm_head)",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": WHOLE_STEP_DRAM_TRAFFIC.get((ctx, model.config.num_hidden_layers)),
                "bytes_per_launch": budget["T"], "us_per_launch": dev_ms * 1e3, "peak_source": peaks["source"],
                "timing": "CUDA events around the %d timed graph replays (one launch each), inputs larger than L2" % steps,
                "isolated_expert_gate_up_kernel": isolated}
        else:
            result["roofline"] = isolated
        result["roofline"]["step_floor_fraction"] = floor_ms / dev_ms
        if not args.no_cpu_baseline and world == 1:
            result["cpu_baseline"] = cpu_baseline_from_session(session, model, spec, ctx, warmup)
    session.close()
    del session
    torch.cuda.empty_cache()
    full_size = args.layers is None
    if not args.no_sub_records and full_size:
        def guarded(fn, *fn_args):
            """A sub-record that fails is reported as such; the headline line is printed whatever happens to them."""
            try:
                return fn(*fn_args)
            except Exception as exc:  # noqa: BLE001
                return {"error": "%s: %s" % (type(exc).__name__, exc)}

        if rank == 0 and ctx != 4096:
            result["ctx4096"] = guarded(sub_ctx4096, model, peaks, device)
        if rank == 0:
            result["config4"] = guarded(sub_config4, peaks)
        barrier()
        ep_rec = guarded(sub_expert_parallel, model, device, world, rank)  # every rank takes part
        if rank == 0:
            result["expert_parallel"] = ep_rec
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        from benchmarks.expert_parallel import shutdown_process_group

        dist.barrier()
        shutdown_process_group()
    return 0


def cpu_baseline_from_session(session, model, spec_bytes, ctx: int, warmup: int) -> dict:
    """The oracle on this box's host cores, same weights (copied from the GPU) and prefilled cache."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from gpu_util import oracle_state_from_session, oracle_weights_from_model
    from oracle import olmoe_decode_oracle as glue

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    spec = glue.OlmoeSpec(layers=model.config.num_hidden_layers)
    session.reset()
    wq = oracle_weights_from_model(model, spec)
    st = oracle_state_from_session(session, spec)
    n = 6
    times = time_oracle_steps(wq, st, session.seed_token_id, ctx, n, 1)
    ms = 1000.0 * sum(times) / len(times)
    return {"value": 1000.0 / ms, "unit": UNIT, "ms_per_step": ms, "cores": torch.get_num_threads(), "kind": "port",
            "sample": "%d greedy decode steps of the same model and prefilled cache on the CPU oracle (1 warm-up)" % n}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--engine", default="auto", choices=["auto", "step", "ops"])
    ap.add_argument("--layers", type=int, default=None, help="decode a model of this many layers instead of 16 (no sub-records)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub-records", action="store_true", help="skip the ctx 4096, isolated-kernel and expert-parallel sub-records")
    ap.add_argument("--step-kernel", default="default", choices=["default", "chained", "whole"],
                    help="step engine: chained kernels with PDL, or the single cooperative whole-step kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.step_kernel != "default":
        from lemoq import _cabi

        _cabi.call("lemoq_set_tuning", 4, 1 if args.step_kernel == "whole" else 0)
    return run_gpu(args)


if __name__ == "__main__":
    raise SystemExit(main())
