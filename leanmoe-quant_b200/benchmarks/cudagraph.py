"""One-token decode session backed by a CUDA graph (reference: benchmarks/cudagraph.py).

Prefill is eager.  The graph holds exactly ONE decode forward and is replayed once per token;
token selection (host ``argmax``) and the position counter stay outside the graph.  Two engines
produce that forward:

``"step"``   the native step engine (``lemoq_step_run``): 6 fused CUDA kernels per layer + lm_head,
             launched from C++ with programmatic dependent launch.  Needs the canonical cell:
             W8 experts, W8 attention projections with packed q.k.v, W8 lm_head, replaced
             attention cores and all fusion switches on (``kv_int8`` may be on or off).
``"ops"``    the model's Python forward with the replaced per-op kernels (any configuration).

``engine="auto"`` takes ``"step"`` when the model qualifies.
"""

from __future__ import annotations

import ctypes
import math
import os
import statistics
import time
from dataclasses import dataclass
from typing import Any

VALID_EXECUTIONS = ("eager", "cudagraph")
VALID_ENGINES = ("auto", "step", "ops")


def normalize_execution(value: str) -> str:
    if value not in VALID_EXECUTIONS:
        raise ValueError("unknown execution %r; expected one of %s" % (value, VALID_EXECUTIONS))
    return value


@dataclass(frozen=True)
class CudaGraphConfig:
    """Static-shape contract of one batch-1 decode graph."""

    ctx: int
    max_new_tokens: int
    batch: int = 1
    q_len: int = 1

    def __post_init__(self) -> None:
        if self.batch != 1:
            raise ValueError("the decode graph supports batch=1 only")
        if self.q_len != 1:
            raise ValueError("the decode graph supports q_len=1 only")
        if self.ctx <= 0 or self.max_new_tokens <= 0:
            raise ValueError("ctx and max_new_tokens must be positive")
        if self.ctx < 2:
            raise ValueError("ctx must be >= 2: ctx=1 routes the prefill token through the q_len=1 decode path "
                             "with filled_len=0 (zero attention)")

    @property
    def max_cache_len(self) -> int:
        return self.ctx + self.max_new_tokens

    def validate_timing(self, timed: int) -> None:
        if timed <= 0:
            raise ValueError("timed must be positive")
        effective = max(timed, 20)
        if effective > self.max_new_tokens:
            raise ValueError("effective timed=%d exceeds max_new_tokens=%d; StaticCache timing horizon would overflow"
                             % (effective, self.max_new_tokens))


@dataclass
class GraphBuffers:
    """Fixed-address step inputs.  ``filled_len`` (int32) is the device-side loop bound of the
    attention kernel; ``cache_position`` (int64) is the slot the new K/V row is written to."""

    token: Any
    cache_position: Any
    position_ids: Any
    attention_mask: Any
    next_token: Any
    filled_len: Any = None
    packed: Any = None  # int64[4] holding token, cache_position, position_ids and (low half of slot 3) filled_len

    @classmethod
    def allocate(cls, device: Any, *, batch: int, max_cache_len: int | None = None, dtype: Any | None = None) -> "GraphBuffers":
        import torch

        if batch != 1:
            raise ValueError("GraphBuffers currently supports batch=1 only")
        max_cache_len = 1 if max_cache_len is None else max_cache_len
        dtype = torch.float32 if dtype is None else dtype
        # The four step scalars are views of ONE 32-byte buffer, so that a caller with host-side inputs can
        # update all of them with a single host->device copy (see pack_step()).
        packed = torch.zeros(4, dtype=torch.long, device=device)
        return cls(
            token=packed[0:1].view(batch, 1),
            cache_position=packed[1:2],
            position_ids=packed[2:3].view(batch, 1),
            attention_mask=torch.zeros((batch, 1, 1, max_cache_len), dtype=dtype, device=device),
            next_token=torch.zeros((batch, 1), dtype=torch.long, device=device),
            filled_len=packed[3:4].view(torch.int32)[0:1],
            packed=packed,
        )

    @staticmethod
    def pack_step(host: Any, *, token: int, position: int) -> Any:
        """Fill a host int64[4] tensor with the image of the step scalars (little-endian int32 in slot 3)."""
        host[0], host[1], host[2], host[3] = int(token), int(position), int(position), int(position) + 1
        return host

    def set_step(self, *, token: int, position: int) -> None:
        self.token.fill_(int(token))
        self.cache_position.fill_(int(position))
        self.position_ids.fill_(int(position))
        if self.filled_len is not None:
            self.filled_len.fill_(int(position) + 1)

    def addresses(self) -> tuple[int, ...]:
        tensors = (self.token, self.cache_position, self.position_ids, self.attention_mask, self.next_token)
        if self.filled_len is not None:
            tensors = tensors + (self.filled_len,)
        return tuple(int(t.data_ptr()) for t in tensors)


class CudaGraphCaptureError(RuntimeError):
    """Capture/replay failure with an explicit lifecycle stage."""

    def __init__(self, stage: str, cause: BaseException):
        self.stage = stage
        self.cause = cause
        super().__init__("CUDA Graph %s failed: %s: %s" % (stage, type(cause).__name__, cause))


class CudaGraphCorrectnessError(CudaGraphCaptureError):
    def __init__(self, report: dict[str, Any]):
        self.report = report
        super().__init__("correctness", RuntimeError("graph/eager correctness gate failed: KL=%s top1=%s"
                                                     % (report.get("kl"), report.get("top1_agreement"))))


def compare_logits(reference: list[Any], candidate: list[Any]) -> dict[str, Any]:
    """Mean over steps of ``KL(ref || got)`` in fp32 and top-1 agreement (both moved to the CPU)."""
    import torch

    if len(reference) != len(candidate) or not reference:
        raise ValueError("reference and candidate must have the same non-empty step count")

    def flat(x: Any) -> Any:
        return x.detach().reshape(1, -1).to(device="cpu", dtype=torch.float32)

    ref = torch.cat([flat(x) for x in reference], dim=0)
    got = torch.cat([flat(x) for x in candidate], dim=0)
    ref_logp, got_logp = torch.log_softmax(ref, dim=-1), torch.log_softmax(got, dim=-1)
    kl = (ref_logp.exp() * (ref_logp - got_logp)).sum(dim=-1).mean()
    agreement = (ref.argmax(dim=-1) == got.argmax(dim=-1)).to(torch.float32).mean()
    return {"kl": max(float(kl.item()), 0.0), "top1_agreement": float(agreement.item())}


def graph_correctness_passed(report: dict[str, Any]) -> bool:
    kl = report.get("kl")
    return bool(kl is not None and math.isfinite(float(kl)) and 0.0 <= float(kl) <= 1e-5
                and report.get("top1_agreement") == 1.0 and report.get("seed_token_match") is True
                and report.get("token_sequence_match") is True)


def replay_timed_step(session: Any) -> Any:
    """One user-visible autoregressive step: step inputs, graph replay, sync, host argmax."""
    return session.replay(synchronize=True)


def summarize(samples: list[float]) -> dict[str, float]:
    s = sorted(samples)
    n = len(s)
    return {"n": n, "p50": statistics.median(s), "p99": s[min(n - 1, int(math.ceil(0.99 * n)) - 1)], "min": s[0],
            "max": s[-1], "mean": sum(s) / n, "stddev": statistics.pstdev(s) if n > 1 else 0.0}


def measure_graph_gap(session: Any, *, warmup: int = 5, timed: int = 20, repeats: int = 3) -> dict[str, Any]:
    """Wall-clock and CUDA-event time per decoded token over ``repeats`` x ``timed`` graph steps,
    each repeat starting from the prefilled state (reset outside the timed window)."""
    torch = session.torch
    warmup, timed = max(warmup, 5), max(timed, 20)
    wall, event = [], []
    for _ in range(repeats):
        session.reset()
        for _ in range(warmup):
            session.replay(synchronize=False)
        session.stream.synchronize()
        session.reset()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(session.stream)
        t0 = time.perf_counter()
        for _ in range(timed):
            replay_timed_step(session)
        session.stream.synchronize()
        wall.append((time.perf_counter() - t0) * 1000.0 / timed)
        end.record(session.stream)
        session.stream.synchronize()
        event.append(start.elapsed_time(end) / timed)
    gpu_only = session.time_graph_only(iters=timed)
    w, e = summarize(wall), summarize(event)
    host = max(w["p50"] - gpu_only, 0.0)
    return {"status": "measured", "method": "perf_counter wall + CUDA events around the greedy loop; back-to-back replays for gpu_busy",
            "wall_p50_ms": w["p50"], "wall_p99_ms": w["p99"], "gpu_p50_ms": e["p50"], "gpu_p99_ms": e["p99"],
            "gpu_busy_ms": gpu_only, "host_p50_ms": host,
            "host_share_pct": round(100.0 * host / w["p50"], 1) if w["p50"] else None,
            "kernels_per_call": session.capture_info.get("kernels_per_step"), "stats": {"wall": w, "gpu_event": e}}


def _skip_mask_fill_enabled() -> bool:
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("skip_mask_fill")


class StaticCacheDecodeSession:
    """Prefill eagerly, capture one decode forward, replay it once per generated token."""

    def __init__(self, model: Any, prompt_ids: Any, *, ctx: int, max_new_tokens: int, device: str = "cuda",
                 engine: str = "auto", use_pdl: bool | None = None, attn_splits: int = 0) -> None:
        import torch

        from lemoq.model import StaticCache

        if engine not in VALID_ENGINES:
            raise ValueError("unknown engine %r; expected one of %s" % (engine, VALID_ENGINES))
        if prompt_ids.ndim != 2 or prompt_ids.shape != (1, ctx):
            raise ValueError("prompt_ids must have shape [1, ctx]")
        self.torch = torch
        self._cuda_available = bool(torch.cuda.is_available())
        self.model = model.eval()
        self.prompt_ids = prompt_ids
        self.device = torch.device(device)
        self.config = CudaGraphConfig(ctx=ctx, max_new_tokens=max_new_tokens, batch=1)
        self.dtype = next(model.parameters()).dtype
        self.cache = StaticCache(config=model.config, max_cache_len=self.config.max_cache_len)
        self.buffers = GraphBuffers.allocate(self.device, batch=1, max_cache_len=self.config.max_cache_len, dtype=self.dtype)
        self.cache._lemoq_filled_len = self.buffers.filled_len
        self.graph = None
        self._captured_mask_independent = False
        self.stream = None
        self.logits = None
        self.current_token_id: int | None = None
        self.position = self.config.ctx
        self.capture_info: dict[str, Any] = {"max_cache_len": self.config.max_cache_len, "q_len": 1, "batch": 1,
                                             "capture_success": False, "replay_success": False}
        env_engine = os.environ.get("LEMOQ_STEP_ENGINE")
        if env_engine is not None and engine == "auto":
            engine = "step" if env_engine == "1" else "ops"
        self._engine_request = engine
        self._use_pdl = (os.environ.get("LEMOQ_PDL", "1") == "1") if use_pdl is None else bool(use_pdl)
        self._attn_splits = int(attn_splits)
        self._step = None  # native step plan (built lazily, after the first prefill)
        self._chain_host = None  # pinned read-back buffer of replay_chained
        self.engine = None
        self.after_prefill = None  # optional callable(session): runs at the end of every prefill
        self.prefill()

    # ------------------------------------------------------------------ prefill
    def _clear_cache(self) -> None:
        self.cache.reset()

    def prefill(self) -> Any:
        """Eagerly fill the static cache and seed the next decode token."""
        torch = self.torch
        self._clear_cache()
        positions = torch.arange(self.config.ctx, device=self.device, dtype=torch.long)
        attention_mask = torch.ones((1, self.config.ctx), device=self.device, dtype=torch.long)
        with torch.no_grad():
            output = self.model(self.prompt_ids, attention_mask=attention_mask, past_key_values=self.cache, use_cache=True,
                                cache_position=positions, position_ids=positions.unsqueeze(0))
        self.current_token_id = int(output.logits[:, -1:, :].argmax(dim=-1).item())
        self.position = self.config.ctx
        if self.after_prefill is not None:
            self.after_prefill(self)
        self._requantize_mirror()
        if self._cuda_available:
            torch.cuda.synchronize()
        return output

    @property
    def seed_token_id(self) -> int:
        if self.current_token_id is None:
            raise RuntimeError("prefill must run before reading the seed token")
        return self.current_token_id

    def buffer_addresses(self) -> tuple[int, ...]:
        return self.buffers.addresses()

    # ------------------------------------------------------------------ engines
    def _step_engine_blocker(self) -> str | None:
        """Why the native step engine cannot serve this model (None = it can)."""
        from lemoq import _cabi
        from lemoq.kernels.fusion_switches import fusion_states
        from lemoq.kernels.moe_grouped_quant import QuantFusedExperts
        from lemoq.quant.linear import QuantLinear

        if not self._cuda_available or self.device.type != "cuda":
            return "no CUDA device"
        if not _cabi.available():
            return _cabi.unavailable_reason()
        if self.dtype != self.torch.float16:
            return "model dtype is not fp16"
        states = fusion_states()
        off = [k for k, v in states.items() if not v and k != "kv_int8"]
        if off:
            return "fusion switches off: %s" % ",".join(sorted(off))
        m = self.model
        if not isinstance(getattr(m, "lm_head", None), QuantLinear):
            return "lm_head is not W8"
        for i, layer in enumerate(m.model.layers):
            attn, mlp = layer.self_attn, layer.mlp
            if getattr(attn, "_lemoq_original_forward", None) is None:
                return "layer %d: attention core not replaced" % i
            if getattr(attn, "_lemoq_packed_qkv", None) is None:
                return "layer %d: packed q/k/v not installed" % i
            if not isinstance(attn.o_proj, QuantLinear):
                return "layer %d: o_proj is not W8" % i
            if not isinstance(getattr(mlp, "_static_experts", None), QuantFusedExperts):
                return "layer %d: experts are not W8 grouped" % i
            if getattr(mlp, "_static_impl", None) != "grouped":
                return "layer %d: MoE impl is not grouped" % i
            if int(getattr(attn, "num_key_value_groups", 1)) != 1:
                return "layer %d: GQA" % i
            if getattr(m.config, "clip_qkv", None) is not None:
                return "clip_qkv is set"
        return None

    def _select_engine(self) -> str:
        if self.engine is not None:
            return self.engine
        blocker = self._step_engine_blocker() if self._engine_request in ("auto", "step") else "engine='ops' requested"
        if blocker is None:
            self.engine = "step"
        elif self._engine_request == "step":
            raise RuntimeError("native step engine unavailable: %s" % blocker)
        else:
            self.engine = "ops"
        self.capture_info["engine"] = self.engine
        self.capture_info["step_engine_blocker"] = blocker
        return self.engine

    def _build_step(self) -> None:
        """Describe the model to the C side once (pointers only; nothing is copied)."""
        from lemoq import _cabi
        from lemoq.kernels.fusion_switches import fusion_enabled
        from lemoq.kernels.kv_int8 import kv_int8_init_buffers

        torch = self.torch
        m, cfg = self.model, self.model.config
        kv_int8 = fusion_enabled("kv_int8")
        max_len = self.config.max_cache_len
        cos, sin = m.model.rotary_emb.tables(max_len, self.dtype, self.device)
        keep: list[Any] = [cos, sin]
        layers = (_cabi.LayerDesc * cfg.num_hidden_layers)()
        for i, layer in enumerate(m.model.layers):
            attn, mlp = layer.self_attn, layer.mlp
            cl = self.cache.layers[i]
            if not cl.is_initialized:
                raise RuntimeError("prefill must run before the step engine is built")
            ex, pk = mlp._static_experts, attn._lemoq_packed_qkv
            d = layers[i]
            d.ln1, d.ln2 = _cabi.ptr(layer.input_layernorm.weight), _cabi.ptr(layer.post_attention_layernorm.weight)
            d.q_norm, d.k_norm = _cabi.ptr(attn.q_norm.weight), _cabi.ptr(attn.k_norm.weight)
            d.qkv_codes, d.qkv_scale = _cabi.ptr(pk.packed), _cabi.ptr(pk.scale)
            d.o_codes, d.o_scale = _cabi.ptr(attn.o_proj.packed), _cabi.ptr(attn.o_proj.scale)
            router = mlp._static_router
            if not router.is_contiguous():
                router = router.contiguous()
                keep.append(router)
            d.router = _cabi.ptr(router)
            d.gu_codes, d.gu_scale = _cabi.ptr(ex.packed_gate_up), _cabi.ptr(ex.scale_gate_up)
            d.dn_codes, d.dn_scale = _cabi.ptr(ex.packed_down), _cabi.ptr(ex.scale_down)
            d.keys, d.values = _cabi.ptr(cl.keys), _cabi.ptr(cl.values)
            if kv_int8:
                bufs = getattr(attn, "_lemoq_kv_int8_bufs", None)
                if bufs is None or tuple(bufs["kc"].shape) != tuple(cl.keys.shape):
                    bufs = kv_int8_init_buffers(cl.keys, cl.values, filled=None)
                    attn._lemoq_kv_int8_bufs = bufs
                import weakref

                attn._lemoq_kv_int8_src_cache_ref = weakref.ref(self.cache)
                d.kc, d.ks, d.vc, d.vs = (_cabi.ptr(bufs[n]) for n in ("kc", "ks", "vc", "vs"))
        desc = _cabi.StepDesc()
        desc.layers, desc.hidden, desc.heads, desc.head_dim = cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim
        desc.experts, desc.top_k, desc.ffn, desc.vocab = cfg.num_experts, cfg.num_experts_per_tok, cfg.intermediate_size, cfg.vocab_size
        desc.group_size = int(m.lm_head.group_size)
        desc.max_len = max_len
        desc.eps = float(cfg.rms_norm_eps)
        desc.norm_topk_prob = int(bool(cfg.norm_topk_prob))
        desc.kv_int8 = int(kv_int8)
        desc.attn_splits = self._attn_splits
        desc.use_pdl = int(self._use_pdl)
        desc.embed = _cabi.ptr(m.model.embed_tokens.weight)
        desc.final_norm = _cabi.ptr(m.model.norm.weight)
        desc.lm_head_codes, desc.lm_head_scale = _cabi.ptr(m.lm_head.packed), _cabi.ptr(m.lm_head.scale)
        desc.rope_cos, desc.rope_sin = _cabi.ptr(cos), _cabi.ptr(sin)
        desc.token, desc.cache_position = _cabi.ptr(self.buffers.token), _cabi.ptr(self.buffers.cache_position)
        desc.filled_len = _cabi.ptr(self.buffers.filled_len)
        logits = torch.zeros((1, 1, cfg.vocab_size), dtype=self.dtype, device=self.device)
        desc.logits = _cabi.ptr(logits)
        next_token = torch.zeros(1, dtype=torch.int64, device=self.device)  # the step's own greedy pick
        desc.next_token = _cabi.ptr(next_token)
        desc.self_feed = 1  # the step leaves its pick, the next slot and the next length in the input scalars
        token_log = torch.zeros(max_len, dtype=torch.int64, device=self.device)  # token_log[position] = the step's pick
        desc.token_log = _cabi.ptr(token_log)
        nbytes = int(_cabi.lib().lemoq_step_workspace_bytes(ctypes.byref(desc)))
        workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        desc.workspace, desc.workspace_bytes = _cabi.ptr(workspace), nbytes
        handle = ctypes.c_void_p()
        _cabi.check(_cabi.lib().lemoq_step_create(ctypes.byref(desc), layers, ctypes.byref(handle)), "lemoq_step_create")
        self._step = {"handle": handle, "logits": logits, "next_token": next_token, "token_log": token_log, "workspace": workspace, "keep": keep, "kv_int8": kv_int8,
                      "desc": desc, "layers": layers}
        self.capture_info["pdl"] = bool(self._use_pdl)

    def _requantize_mirror(self) -> None:
        """After a (re)prefill: rebuild, in place, every int8 mirror that was built from this
        session's cache (both engines keep it on the attention module), so slots written by earlier
        decode steps cannot leak into the next sequence."""
        if not self._cuda_available:
            return
        from lemoq import _cabi

        stream = None
        for i, layer in enumerate(self.model.model.layers):
            attn = getattr(layer, "self_attn", None)
            bufs = getattr(attn, "_lemoq_kv_int8_bufs", None)
            ref = getattr(attn, "_lemoq_kv_int8_src_cache_ref", None)
            cl = self.cache.layers[i]
            if bufs is None or ref is None or ref() is not self.cache or not cl.is_initialized:
                continue
            if tuple(bufs["kc"].shape) != tuple(cl.keys.shape):
                continue
            stream = _cabi.current_stream(self.device) if stream is None else stream
            _, h, s, d = (int(v) for v in cl.keys.shape)
            _cabi.call("lemoq_kv_int8_bulk_quantize", _cabi.ptr(cl.keys), _cabi.ptr(cl.values), _cabi.ptr(bufs["kc"]),
                       _cabi.ptr(bufs["ks"]), _cabi.ptr(bufs["vc"]), _cabi.ptr(bufs["vs"]), h, s, d, -1, stream)

    def _forward_once(self) -> Any:
        """Enqueue one decode forward on the current stream; returns the logits tensor."""
        if self._select_engine() == "step":
            from lemoq import _cabi

            if self._step is None:
                self._build_step()
            n = ctypes.c_int(0)
            _cabi.check(_cabi.lib().lemoq_step_run(self._step["handle"], _cabi.current_stream(self.device), ctypes.byref(n)),
                        "lemoq_step_run")
            self.capture_info["kernels_per_step"] = int(n.value)
            self.capture_info["step_kernel"] = _cabi.lib().lemoq_step_engine(self._step["handle"]).decode()
            return self._step["logits"]
        output = self.model(self.buffers.token, attention_mask=self.buffers.attention_mask, past_key_values=self.cache,
                            use_cache=True, cache_position=self.buffers.cache_position, position_ids=self.buffers.position_ids)
        return output.logits

    def step_error_flags(self) -> int:
        """Bit mask set by a kernel that had to clamp a position / length / expert id (0 = clean)."""
        if self._step is None:
            return 0
        from lemoq import _cabi

        addr = _cabi.lib().lemoq_step_error_flag(self._step["handle"])
        off = int(addr) - int(self._step["workspace"].data_ptr())
        self.torch.cuda.synchronize()
        return int(self._step["workspace"][off: off + 4].view(self.torch.int32).item())

    def step_topk_ids(self) -> Any:
        """``(layers, top_k)`` int64 expert ids chosen in the most recent step (step engine only)."""
        if self._step is None:
            raise RuntimeError("the step engine has not run")
        from lemoq import _cabi

        cfg = self.model.config
        addr = _cabi.lib().lemoq_step_topk_ids(self._step["handle"])
        off = int(addr) - int(self._step["workspace"].data_ptr())
        n = cfg.num_hidden_layers * cfg.num_experts_per_tok
        self.torch.cuda.synchronize()
        return self._step["workspace"][off: off + 8 * n].view(self.torch.int64).reshape(cfg.num_hidden_layers, -1).clone()

    def step_router_logits(self) -> Any:
        """``(layers, experts)`` fp16 router logits of the most recent step (step engine only)."""
        if self._step is None:
            raise RuntimeError("the step engine has not run")
        from lemoq import _cabi

        cfg = self.model.config
        addr = _cabi.lib().lemoq_step_router_logits(self._step["handle"])
        off = int(addr) - int(self._step["workspace"].data_ptr())
        n = cfg.num_hidden_layers * cfg.num_experts
        self.torch.cuda.synchronize()
        return self._step["workspace"][off: off + 2 * n].view(self.torch.float16).reshape(cfg.num_hidden_layers, -1).clone()

    @property
    def step_next_token(self) -> Any:
        """Device scalar holding the token the native step engine picked in its last step (None for the per-op engine)."""
        if self._step is None or self.capture_info.get("engine") != "step":
            return None
        return self._step["next_token"]

    def step_phase_times_us(self) -> Any:
        """Per-phase durations (us) of the last whole-step kernel: a (layers, 6) tensor for the phases
        q.k.v / attention / o_proj / router / gate_up / down plus the lm_head time; None when the step
        runs as chained kernels."""
        if self._step is None:
            return None
        from lemoq import _cabi

        addr = _cabi.lib().lemoq_step_phase_stamps(self._step["handle"])
        if not addr:
            return None
        layers = self.model.config.num_hidden_layers
        off = int(addr) - int(self._step["workspace"].data_ptr())
        self.torch.cuda.synchronize()
        st = self._step["workspace"][off: off + 8 * (6 * layers + 2)].view(self.torch.int64).cpu().double()
        d = (st[1:] - st[:-1]) / 1000.0
        return {"phases": d[: 6 * layers].reshape(layers, 6), "lm_head": float(d[6 * layers]), "total": float((st[-1] - st[0]) / 1000.0)}

    # ------------------------------------------------------------------ decode
    def decode_eager(self) -> Any:
        if self.current_token_id is None:
            raise RuntimeError("prefill must run before decode")
        if self.position >= self.config.max_cache_len:
            raise RuntimeError("decode position exceeded StaticCache capacity")
        self._set_step_inputs()
        with self.torch.no_grad():
            logits = self._forward_once().detach()
        self.current_token_id = int(logits.reshape(-1).argmax().item())
        self.position += 1
        if self._cuda_available:
            self.torch.cuda.synchronize()
        return logits

    def _decode_mask_independent(self) -> bool:
        if self.engine == "step":
            return True
        from lemoq.kernels.attn_decode import _decode_forward_impl

        config = getattr(self.model, "config", None)
        if getattr(config, "model_type", None) != "olmoe" or getattr(config, "output_attentions", False):
            return False
        layers = getattr(getattr(self.model, "model", None), "layers", ())
        if not layers:
            return False
        for layer in layers:
            attn = getattr(layer, "self_attn", None)
            if (getattr(attn, "_lemoq_attn_backend", None) not in ("cuda", "triton")
                    or getattr(getattr(attn, "forward", None), "__func__", None) is not _decode_forward_impl
                    or getattr(attn, "num_key_value_groups", 1) != 1):
                return False
        return True

    def _set_step_inputs(self, *, skip_mask: bool = False) -> None:
        if skip_mask and not getattr(self, "_captured_mask_independent", False):
            raise RuntimeError("skip-mask-fill requires a captured mask-independent kernel backend")
        if self.current_token_id is None:
            raise RuntimeError("prefill must run before decode")
        if self.position >= self.config.max_cache_len:
            raise RuntimeError("decode position exceeded StaticCache capacity")
        torch = self.torch
        self.buffers.token.fill_(self.current_token_id)
        self.buffers.cache_position.fill_(self.position)
        self.buffers.position_ids.fill_(self.position)
        if not skip_mask:
            self.buffers.attention_mask.fill_(torch.finfo(self.dtype).min)
            self.buffers.attention_mask[..., : self.position + 1].zero_()
        self.buffers.filled_len.fill_(self.position + 1)

    def capture(self, *, warmup: int = 5) -> dict[str, Any]:
        """Warm up eagerly on a side stream, restore the prefilled state, capture one forward."""
        torch = self.torch
        if self.graph is not None:
            return dict(self.capture_info)
        if warmup < 1:
            raise ValueError("warmup must be positive")
        try:
            self.prefill()
            self.stream = torch.cuda.Stream(device=self.device)
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            initial_token, initial_position = self.current_token_id, self.position
            with torch.cuda.stream(self.stream), torch.no_grad():
                for _ in range(warmup):
                    self._set_step_inputs()
                    self._forward_once()
            self.stream.synchronize()
            self.prefill()
            self.current_token_id, self.position = initial_token, initial_position
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self._set_step_inputs()
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream), torch.no_grad():
                self.logits = self._forward_once()
            self.stream.synchronize()
            self.graph = graph
            self._captured_mask_independent = self._decode_mask_independent()
            self.capture_info.update(mask_independent_decode=self._captured_mask_independent, capture_success=True,
                                     stream="dedicated CUDA stream")
            return dict(self.capture_info)
        except Exception as exc:  # noqa: BLE001
            raise CudaGraphCaptureError("capture", exc) from exc

    def _replay_skip_mask(self) -> bool:
        return _skip_mask_fill_enabled() and self._captured_mask_independent

    def replay(self, *, synchronize: bool = True) -> Any:
        """Replay one decode step; with ``synchronize`` also pick the next token and advance."""
        if self.graph is None or self.stream is None or self.logits is None:
            raise RuntimeError("capture must succeed before replay")
        try:
            with self.torch.cuda.stream(self.stream), self.torch.no_grad():
                self._set_step_inputs(skip_mask=self._replay_skip_mask())
                self.graph.replay()
            if synchronize:
                self.stream.synchronize()
                picked = self.step_next_token
                # the native step engine picks the token itself (first maximal logit, like a host arg-max)
                self.current_token_id = int(picked.item()) if picked is not None else int(self.logits.reshape(-1).argmax().item())
                self.position += 1
            self.capture_info["replay_success"] = True
            return self.logits
        except Exception as exc:  # noqa: BLE001
            raise CudaGraphCaptureError("replay", exc) from exc

    def replay_chained(self, steps: int) -> list[int]:
        """``steps`` greedy decode steps with no host work in between (native step engine only): the step inputs go to
        the device once, every replay leaves its pick, the next slot and the next length in the input scalars for the
        next one and logs its token; one read-back of ``steps`` token ids at the end.  Replaces ``steps`` rounds of the
        reference's set-inputs / replay / synchronize / read-back loop (benchmarks/cudagraph.py:756-762)."""
        if self.graph is None or self._step is None or self.capture_info.get("engine") != "step":
            raise RuntimeError("replay_chained needs the captured native step engine")
        if steps <= 0:
            raise ValueError("steps must be positive")
        if self.position + steps > self.config.max_cache_len:
            raise RuntimeError("replay_chained: exceeded StaticCache capacity (%d + %d > %d)"
                               % (self.position, steps, self.config.max_cache_len))
        torch = self.torch
        if self._chain_host is None or self._chain_host.numel() < steps + 4:
            self._chain_host = torch.zeros(max(steps, 64) + 4, dtype=torch.int64).pin_memory()
        if self.current_token_id is None:
            raise RuntimeError("prefill must run before decode")
        try:
            with torch.cuda.stream(self.stream), torch.no_grad():
                # the step scalars of the first step: one 32-byte copy from pinned host memory into the packed buffer
                host_in = self.buffers.pack_step(self._chain_host[-4:], token=self.current_token_id, position=self.position)
                self.buffers.packed.copy_(host_in, non_blocking=True)
                for _ in range(steps):
                    self.graph.replay()
                log = self._step["token_log"][self.position: self.position + steps]
                self._chain_host[:steps].copy_(log, non_blocking=True)
            self.stream.synchronize()
        except Exception as exc:  # noqa: BLE001
            raise CudaGraphCaptureError("replay", exc) from exc
        tokens = [int(v) for v in self._chain_host[:steps].tolist()]
        self.position += steps
        self.current_token_id = tokens[-1]
        return tokens

    def set_position(self, position: int) -> None:
        if position < 0 or position >= self.config.max_cache_len:
            raise RuntimeError("position %d 超出 StaticCache 容量 %d" % (position, self.config.max_cache_len))
        self.position = int(position)

    def replay_at_position(self, position: int, *, synchronize: bool = True) -> Any:
        self.set_position(position)
        return self.replay(synchronize=synchronize)

    def time_graph_only(self, iters: int = 20) -> float:
        """Mean device time (ms) of back-to-back graph replays at the current position, no host work
        in between (CUDA events on the session stream)."""
        torch = self.torch
        if self.graph is None:
            raise RuntimeError("capture must succeed before timing")
        saved = self.position
        if self._step is not None:  # the native step advances its own position: stay inside the cache
            self.position = max(0, min(self.position, self.config.max_cache_len - iters - 4))
        with torch.cuda.stream(self.stream):
            self._set_step_inputs(skip_mask=self._replay_skip_mask())
            self.position = saved
            for _ in range(3):
                self.graph.replay()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(self.stream)
            for _ in range(iters):
                self.graph.replay()
            end.record(self.stream)
        self.stream.synchronize()
        return start.elapsed_time(end) / iters

    def logits_cpu(self) -> Any:
        if self.stream is None or self.logits is None:
            raise RuntimeError("no graph output is available")
        self.stream.synchronize()
        return self.logits.detach().to("cpu").clone()

    def next_token_cpu(self) -> int:
        if self.stream is None or self.current_token_id is None:
            raise RuntimeError("no graph output is available")
        self.stream.synchronize()
        return self.current_token_id

    def reset(self) -> None:
        self.prefill()

    def close(self) -> None:
        if self._step is not None:
            from lemoq import _cabi

            _cabi.lib().lemoq_step_destroy(self._step["handle"])
            self._step = None
