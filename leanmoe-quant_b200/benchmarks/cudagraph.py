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
_MIN_TIMED = 20   # a timing run never uses fewer steps than this ...
_MIN_WARMUP = 5   # ... nor fewer warm-up steps
_KL_GATE = 1e-5   # graph replay against the same path run eagerly


def _one_of(value: str, allowed: tuple[str, ...], what: str) -> str:
    if value not in allowed:
        raise ValueError("unknown %s %r; expected one of %s" % (what, value, allowed))
    return value


def normalize_execution(value: str) -> str:
    return _one_of(value, VALID_EXECUTIONS, "execution")


@dataclass(frozen=True)
class CudaGraphConfig:
    """The fixed shape of one batch-1 decode graph: prompt length, room for new tokens, one row, one query."""

    ctx: int
    max_new_tokens: int
    batch: int = 1
    q_len: int = 1

    def __post_init__(self) -> None:
        for ok, text in (
            (self.batch == 1, "the decode graph supports batch=1 only"),
            (self.q_len == 1, "the decode graph supports q_len=1 only"),
            (self.ctx > 0 and self.max_new_tokens > 0, "ctx and max_new_tokens must be positive"),
            # with ctx=1 the prompt itself would go through the one-token path with nothing filled yet
            (self.ctx >= 2, "ctx must be >= 2: ctx=1 routes the prefill token through the q_len=1 decode path "
                            "with filled_len=0 (zero attention)"),
        ):
            if not ok:
                raise ValueError(text)

    @property
    def max_cache_len(self) -> int:
        return self.ctx + self.max_new_tokens

    def validate_timing(self, timed: int) -> None:
        """A timing run of ``timed`` steps (at least ``_MIN_TIMED`` are run) must fit into the room for new tokens."""
        if timed <= 0:
            raise ValueError("timed must be positive")
        run = max(timed, _MIN_TIMED)
        if run > self.max_new_tokens:
            raise ValueError("effective timed=%d exceeds max_new_tokens=%d; StaticCache timing horizon would overflow"
                             % (run, self.max_new_tokens))


@dataclass
class GraphBuffers:
    """The step inputs at addresses that never change.  ``token``, ``cache_position`` (the slot the new key/value row
    goes to), ``position_ids`` and ``filled_len`` (int32: the attention kernel's loop bound) are views of ONE
    ``int64[4]`` array, ``packed``, so a host-driven loop updates all four with a single 32-byte copy."""

    token: Any
    cache_position: Any
    position_ids: Any
    attention_mask: Any
    next_token: Any
    filled_len: Any = None
    packed: Any = None

    @classmethod
    def allocate(cls, device: Any, *, batch: int, max_cache_len: int | None = None, dtype: Any | None = None) -> "GraphBuffers":
        import torch

        if batch != 1:
            raise ValueError("GraphBuffers currently supports batch=1 only")
        words = torch.zeros(4, dtype=torch.long, device=device)
        mask = torch.zeros((1, 1, 1, max_cache_len or 1), dtype=dtype or torch.float32, device=device)
        return cls(token=words[0:1].view(1, 1), cache_position=words[1:2], position_ids=words[2:3].view(1, 1),
                   attention_mask=mask, next_token=torch.zeros((1, 1), dtype=torch.long, device=device),
                   filled_len=words[3:4].view(torch.int32)[0:1], packed=words)

    @staticmethod
    def pack_step(host: Any, *, token: int, position: int) -> Any:
        """The image of the four scalars for (``token``, ``position``) in a host ``int64[4]``: the length
        ``position + 1`` sits in the low half of word 3 (little-endian)."""
        for word, value in enumerate((token, position, position, position + 1)):
            host[word] = int(value)
        return host

    def set_step(self, *, token: int, position: int) -> None:
        self.token.fill_(int(token))
        for scalar in (self.cache_position, self.position_ids):
            scalar.fill_(int(position))
        if self.filled_len is not None:
            self.filled_len.fill_(int(position) + 1)

    def addresses(self) -> tuple[int, ...]:
        """Device addresses of the inputs (a replay must find them where capture saw them)."""
        fixed = [self.token, self.cache_position, self.position_ids, self.attention_mask, self.next_token]
        fixed += [] if self.filled_len is None else [self.filled_len]
        return tuple(int(t.data_ptr()) for t in fixed)


class CudaGraphCaptureError(RuntimeError):
    """A failure in ``stage`` ("capture", "replay", "correctness") of the graph's life; ``cause`` is the original."""

    def __init__(self, stage: str, cause: BaseException):
        super().__init__("CUDA Graph %s failed: %s: %s" % (stage, type(cause).__name__, cause))
        self.stage, self.cause = stage, cause


class CudaGraphCorrectnessError(CudaGraphCaptureError):
    def __init__(self, report: dict[str, Any]):
        summary = "graph/eager correctness gate failed: KL=%s top1=%s" % (report.get("kl"), report.get("top1_agreement"))
        super().__init__("correctness", RuntimeError(summary))
        self.report = report


def compare_logits(reference: list[Any], candidate: list[Any]) -> dict[str, Any]:
    """``KL(reference || candidate)`` averaged over the steps, and the share of steps with the same arg-max.
    Computed on the CPU in fp32 whatever the inputs are."""
    import torch

    if not reference or len(reference) != len(candidate):
        raise ValueError("reference and candidate must have the same non-empty step count")
    rows = lambda steps: torch.stack([t.detach().reshape(-1).to("cpu", torch.float32) for t in steps])  # noqa: E731
    ref, got = rows(reference), rows(candidate)
    log_p, log_q = ref.log_softmax(-1), got.log_softmax(-1)
    kl = torch.sum(log_p.exp() * (log_p - log_q), dim=-1).mean().item()
    same = (ref.argmax(-1) == got.argmax(-1)).float().mean().item()
    return {"kl": max(float(kl), 0.0), "top1_agreement": float(same)}


def graph_correctness_passed(report: dict[str, Any]) -> bool:
    """The gate of graph replay against eager: KL within ``_KL_GATE`` (and finite), every arg-max equal, the same seed
    token and the same token sequence."""
    kl = report.get("kl")
    if kl is None or not math.isfinite(float(kl)) or not 0.0 <= float(kl) <= _KL_GATE:
        return False
    return report.get("top1_agreement") == 1.0 and all(report.get(k) is True for k in ("seed_token_match", "token_sequence_match"))


def replay_timed_step(session: Any) -> Any:
    """What one generated token costs a user: set the inputs, replay, synchronize, pick the next token."""
    return session.replay(synchronize=True)


def summarize(samples: list[float]) -> dict[str, float]:
    ordered = sorted(samples)
    count = len(ordered)
    rank99 = min(count, max(1, math.ceil(0.99 * count)))  # nearest-rank percentile
    return {"n": count, "p50": statistics.median(ordered), "p99": ordered[rank99 - 1], "min": ordered[0], "max": ordered[-1],
            "mean": math.fsum(ordered) / count, "stddev": statistics.pstdev(ordered) if count > 1 else 0.0}


def measure_graph_gap(session: Any, *, warmup: int = 5, timed: int = 20, repeats: int = 3) -> dict[str, Any]:
    """Per generated token: wall-clock and CUDA-event time of the host-driven greedy loop (``repeats`` runs of ``timed``
    steps, each from the prefilled state, resets outside the timed window), against the device time of back-to-back
    replays.  The difference is what the host costs."""
    torch = session.torch
    warmup, timed = max(warmup, _MIN_WARMUP), max(timed, _MIN_TIMED)
    wall_ms, event_ms = [], []
    for _ in range(repeats):
        session.reset()
        for _ in range(warmup):
            session.replay(synchronize=False)
        session.stream.synchronize()
        session.reset()
        first, last = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        first.record(session.stream)
        began = time.perf_counter()
        for _ in range(timed):
            replay_timed_step(session)
        session.stream.synchronize()
        wall_ms.append(1e3 * (time.perf_counter() - began) / timed)
        last.record(session.stream)
        session.stream.synchronize()
        event_ms.append(first.elapsed_time(last) / timed)
    busy = session.time_graph_only(iters=timed)
    wall, event = summarize(wall_ms), summarize(event_ms)
    host = max(wall["p50"] - busy, 0.0)
    return {"status": "measured", "method": "perf_counter wall + CUDA events around the greedy loop; back-to-back replays for gpu_busy",
            "wall_p50_ms": wall["p50"], "wall_p99_ms": wall["p99"], "gpu_p50_ms": event["p50"], "gpu_p99_ms": event["p99"],
            "gpu_busy_ms": busy, "host_p50_ms": host, "host_share_pct": round(100.0 * host / wall["p50"], 1) if wall["p50"] else None,
            "kernels_per_call": session.capture_info.get("kernels_per_step"), "stats": {"wall": wall, "gpu_event": event}}


def _skip_mask_fill_enabled() -> bool:
    from lemoq.kernels.fusion_switches import fusion_enabled

    return fusion_enabled("skip_mask_fill")


class StaticCacheDecodeSession:
    """Prefill eagerly, capture one decode forward, replay it once per generated token."""

    def __init__(self, model: Any, prompt_ids: Any, *, ctx: int, max_new_tokens: int, device: str = "cuda",
                 engine: str = "auto", use_pdl: bool | None = None, attn_splits: int = 0) -> None:
        import torch

        from lemoq.model import StaticCache

        _one_of(engine, VALID_ENGINES, "engine")
        if tuple(prompt_ids.shape) != (1, ctx):
            raise ValueError("prompt_ids must have shape [1, ctx]")
        self.torch = torch
        self.device = torch.device(device)
        self._cuda_available = bool(torch.cuda.is_available())
        self.config = CudaGraphConfig(ctx=ctx, max_new_tokens=max_new_tokens, batch=1)
        self.model, self.prompt_ids = model.eval(), prompt_ids
        self.dtype = next(model.parameters()).dtype
        capacity = self.config.max_cache_len
        self.cache = StaticCache(config=model.config, max_cache_len=capacity)
        self.buffers = GraphBuffers.allocate(self.device, batch=1, max_cache_len=capacity, dtype=self.dtype)
        self.cache._lemoq_filled_len = self.buffers.filled_len  # the attention modules find the device length here
        # engine choice: an explicit argument wins; "auto" listens to LEMOQ_STEP_ENGINE (1 = step, else ops)
        forced = os.environ.get("LEMOQ_STEP_ENGINE")
        self._engine_request = engine if engine != "auto" or forced is None else ("step" if forced == "1" else "ops")
        self._use_pdl = os.environ.get("LEMOQ_PDL", "1") == "1" if use_pdl is None else bool(use_pdl)
        self._attn_splits = int(attn_splits)
        self.engine = None
        self._step = None         # plan of the native step engine (built after the first prefill)
        self._chain_host = None   # pinned buffer of replay_chained
        self.after_prefill = None  # optional callable(session), run at the end of every prefill
        # graph state
        self.graph = self.stream = self.logits = None
        self._captured_mask_independent = False
        self.capture_info: dict[str, Any] = {"max_cache_len": capacity, "q_len": 1, "batch": 1, "capture_success": False,
                                             "replay_success": False}
        # decode state
        self.current_token_id: int | None = None
        self.position = ctx
        self.prefill()

    # ------------------------------------------------------------------ prefill
    def _clear_cache(self) -> None:
        self.cache.reset()

    def prefill(self) -> Any:
        """Run the prompt through the model eagerly into the emptied static cache; the arg-max of the last position
        seeds the decode."""
        torch, ctx = self.torch, self.config.ctx
        self._clear_cache()
        slots = torch.arange(ctx, dtype=torch.long, device=self.device)
        with torch.no_grad():
            output = self.model(self.prompt_ids, attention_mask=torch.ones_like(slots).unsqueeze(0), past_key_values=self.cache,
                                use_cache=True, cache_position=slots, position_ids=slots.unsqueeze(0))
        self.current_token_id, self.position = int(output.logits[0, -1].argmax().item()), ctx
        if self.after_prefill is not None:
            self.after_prefill(self)
        self._requantize_mirror()
        self._device_sync()
        return output

    def _device_sync(self) -> None:
        if self._cuda_available:
            self.torch.cuda.synchronize()

    def _seeded_token(self, purpose: str) -> int:
        if self.current_token_id is None:
            raise RuntimeError("prefill must run before %s" % purpose)
        return self.current_token_id

    def _room_for(self, steps: int = 1) -> None:
        if self.position + steps > self.config.max_cache_len:
            raise RuntimeError("decode position exceeded StaticCache capacity (%d + %d > %d)"
                               % (self.position, steps, self.config.max_cache_len))

    @property
    def seed_token_id(self) -> int:
        return self._seeded_token("reading the seed token")

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

    def clear_step_error_flags(self) -> None:
        """Zero the step engine's flag word (the flags are sticky: a step never clears what an earlier one raised)."""
        if self._step is None:
            return
        from lemoq import _cabi

        addr = _cabi.lib().lemoq_step_error_flag(self._step["handle"])
        off = int(addr) - int(self._step["workspace"].data_ptr())
        self.torch.cuda.synchronize()
        self._step["workspace"][off: off + 4].zero_()

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
    def _adopt(self, logits: Any) -> None:
        """Take the step's pick as the next input.  The native step engine has picked on the device (first maximal
        logit, which is what a host arg-max returns); otherwise pick here."""
        picked = self.step_next_token
        self.current_token_id = int((picked if picked is not None else logits.reshape(-1).argmax()).item())
        self.position += 1

    def decode_eager(self) -> Any:
        """One decode step without the graph (the comparison arm of the correctness gate)."""
        self._set_step_inputs()
        with self.torch.no_grad():
            logits = self._forward_once().detach()
        self._device_sync()
        self.current_token_id = int(logits.reshape(-1).argmax().item())
        self.position += 1
        return logits

    def _decode_mask_independent(self) -> bool:
        """Does the captured forward ignore ``attention_mask``?  True for the native step engine, and for the Python
        forward when EVERY layer's attention is the patched decode kernel (no grouped-query heads): then the
        per-step mask fill can be left out."""
        if self.engine == "step":
            return True
        from lemoq.kernels.attn_decode import _decode_forward_impl

        config = getattr(self.model, "config", None)
        decoder_layers = getattr(getattr(self.model, "model", None), "layers", None) or ()
        if getattr(config, "model_type", None) != "olmoe" or getattr(config, "output_attentions", False) or not decoder_layers:
            return False

        def kernel_attention(attn: Any) -> bool:
            bound_to = getattr(getattr(attn, "forward", None), "__func__", None)
            return (bound_to is _decode_forward_impl and getattr(attn, "_lemoq_attn_backend", None) in ("cuda", "triton")
                    and getattr(attn, "num_key_value_groups", 1) == 1)

        return all(kernel_attention(getattr(layer, "self_attn", None)) for layer in decoder_layers)

    def _set_step_inputs(self, *, skip_mask: bool = False) -> None:
        """Write token, slot, position and length of the current step into the fixed buffers, and (unless skipped)
        the additive mask that opens positions ``[0, position]``."""
        if skip_mask and not getattr(self, "_captured_mask_independent", False):
            raise RuntimeError("skip-mask-fill requires a captured mask-independent kernel backend")
        token = self._seeded_token("decode")
        self._room_for(1)
        self.buffers.set_step(token=token, position=self.position)
        if not skip_mask:
            mask = self.buffers.attention_mask
            mask.fill_(self.torch.finfo(self.dtype).min)
            mask[..., : self.position + 1] = 0

    def capture(self, *, warmup: int = 5) -> dict[str, Any]:
        """Capture ONE decode forward on a stream of its own.  Before that: ``warmup`` eager steps on that stream (they
        create every lazily built buffer), then a fresh prefill so the captured state is the prefilled one."""
        if self.graph is not None:
            return dict(self.capture_info)
        if warmup < 1:
            raise ValueError("warmup must be positive")
        torch = self.torch
        try:
            self.prefill()
            seed = (self.current_token_id, self.position)
            side = self.stream = torch.cuda.Stream(device=self.device)
            main = torch.cuda.current_stream(self.device)
            side.wait_stream(main)
            with torch.cuda.stream(side), torch.no_grad():
                for _ in range(warmup):  # same inputs every time: the steps only have to run, not to advance
                    self._set_step_inputs()
                    self._forward_once()
            side.synchronize()
            self.prefill()
            self.current_token_id, self.position = seed
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self._set_step_inputs()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side), torch.no_grad():
                self.logits = self._forward_once()
            side.synchronize()
        except Exception as exc:  # noqa: BLE001 - every failure is reported with its stage
            raise CudaGraphCaptureError("capture", exc) from exc
        self.graph = graph
        self._captured_mask_independent = self._decode_mask_independent()
        self.capture_info.update(capture_success=True, stream="dedicated CUDA stream",
                                 mask_independent_decode=self._captured_mask_independent)
        return dict(self.capture_info)

    def _replay_skip_mask(self) -> bool:
        return self._captured_mask_independent and _skip_mask_fill_enabled()

    def _captured(self, purpose: str) -> None:
        if self.graph is None or self.stream is None or self.logits is None:
            raise RuntimeError("capture must succeed before %s" % purpose)

    def replay(self, *, synchronize: bool = True) -> Any:
        """One decode step through the graph.  With ``synchronize`` the host waits, adopts the pick and advances;
        without, it only queues the step (same inputs next time)."""
        self._captured("replay")
        try:
            with self.torch.cuda.stream(self.stream), self.torch.no_grad():
                self._set_step_inputs(skip_mask=self._replay_skip_mask())
                self.graph.replay()
            if synchronize:
                self.stream.synchronize()
                self._adopt(self.logits)
        except Exception as exc:  # noqa: BLE001
            raise CudaGraphCaptureError("replay", exc) from exc
        self.capture_info["replay_success"] = True
        return self.logits

    def replay_chained(self, steps: int) -> list[int]:
        """``steps`` greedy decode steps with no host work in between (native step engine only): the step inputs go to
        the device once, every replay leaves its pick, the next slot and the next length in the input scalars for the
        next one and logs its token; one read-back of ``steps`` token ids at the end.  Replaces ``steps`` rounds of the
        reference's set-inputs / replay / synchronize / read-back loop (benchmarks/cudagraph.py:756-762)."""
        if self.graph is None or self._step is None or self.capture_info.get("engine") != "step":
            raise RuntimeError("replay_chained needs the captured native step engine")
        if steps <= 0:
            raise ValueError("steps must be positive")
        first_token = self._seeded_token("decode")
        self._room_for(steps)
        torch = self.torch
        if self._chain_host is None or self._chain_host.numel() < steps + 4:
            self._chain_host = torch.zeros(max(steps, 64) + 4, dtype=torch.int64).pin_memory()
        scalars, tokens_out = self._chain_host[-4:], self._chain_host[:steps]
        try:
            with torch.cuda.stream(self.stream), torch.no_grad():
                # the first step's scalars: one 32-byte copy from pinned host memory into the packed buffer
                self.buffers.packed.copy_(self.buffers.pack_step(scalars, token=first_token, position=self.position), non_blocking=True)
                for _ in range(steps):
                    self.graph.replay()
                tokens_out.copy_(self._step["token_log"][self.position: self.position + steps], non_blocking=True)
            self.stream.synchronize()
        except Exception as exc:  # noqa: BLE001
            raise CudaGraphCaptureError("replay", exc) from exc
        tokens = [int(t) for t in tokens_out.tolist()]
        self.position += steps
        self.current_token_id = tokens[-1]
        return tokens

    def set_position(self, position: int) -> None:
        if not 0 <= position < self.config.max_cache_len:
            raise RuntimeError("position %d 超出 StaticCache 容量 %d (outside the cache)" % (position, self.config.max_cache_len))
        self.position = int(position)

    def replay_at_position(self, position: int, *, synchronize: bool = True) -> Any:
        self.set_position(position)
        return self.replay(synchronize=synchronize)

    def time_graph_only(self, iters: int = 20) -> float:
        """Mean device time (ms) of ``iters`` back-to-back replays with no host work between them, from CUDA events on
        the session's stream.  The session's position is left as it was."""
        if self.graph is None:
            raise RuntimeError("capture must succeed before timing")
        torch, here = self.torch, self.position
        if self._step is not None:  # the native step advances its own position: start where iters + warm-up still fit
            self.position = max(0, min(here, self.config.max_cache_len - iters - 4))
        first, last = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        with torch.cuda.stream(self.stream):
            self._set_step_inputs(skip_mask=self._replay_skip_mask())
            self.position = here
            for i in range(3 + iters):
                if i == 3:
                    first.record(self.stream)
                self.graph.replay()
            last.record(self.stream)
        self.stream.synchronize()
        return first.elapsed_time(last) / iters

    def _graph_output(self, value: Any) -> Any:
        if self.stream is None or value is None:
            raise RuntimeError("no graph output is available")
        self.stream.synchronize()
        return value

    def logits_cpu(self) -> Any:
        return self._graph_output(self.logits).detach().cpu().clone()

    def next_token_cpu(self) -> int:
        return self._graph_output(self.current_token_id)

    def reset(self) -> None:
        self.prefill()

    def close(self) -> None:
        if self._step is not None:
            from lemoq import _cabi

            _cabi.lib().lemoq_step_destroy(self._step["handle"])
            self._step = None
