"""Batched expert-parallel decode (benchmark configuration 5): B sequences in lockstep, the attention/dense part
data-parallel over the sequences (weights replicated, every rank owns B/G sequences and their int8 KV),
the MoE expert-parallel (expert e lives on rank e // (E/G)).

Per layer and rank:  route the local tokens -> **all-to-all dispatch** of the (token, slot) pairs to the
ranks that own their experts (fp16 activation row + global expert id, pairs sorted by expert so that a
rank streams each resident expert's weights once) -> grouped expert GEMV on the received pairs ->
**all-to-all combine** of the fp16 expert outputs -> routing-weighted sum at the home rank in slot order
(fp32, one rounding) + residual.  Two all-to-alls per layer over NCCL (NVLink/NVSwitch), 32 per step.  Two forms of
the exchange: **static** (default) sends every peer a fixed number of pair slots, reads nothing on the host and is
captured, all-to-alls included, in one CUDA graph; **dynamic** exchanges the pair counts first and reads them on the
host.  Buffers are received into local memory before any kernel touches them; no peer pointers.

There is no counterpart in the reference (its runner is batch 1, `benchmarks/runner.py`); the oracle for
this mode is the same decoder at world size 1: results must match it token for token, which the
dispatch/combine guarantees because every pair's expert output is computed by the same kernel on the
same inputs whichever rank owns the expert, and the combine order is the slot order.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 --master-port P \
        leanmoe-quant_b200/benchmarks/expert_parallel.py --sequences 64 --ctx 2048 --steps 32
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from dataclasses import dataclass
from typing import Any, Callable

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _PKG not in sys.path:
    sys.path.insert(0, _PKG)

import torch  # noqa: E402


# ---------------------------------------------------------------------------------------------------
# dispatch / combine (device-agnostic tensor logic + torch.distributed; tested with gloo on CPU)
# ---------------------------------------------------------------------------------------------------
@dataclass
class DispatchPlan:
    order: Any          # (P,) pair indices (t*K + k) sorted by global expert id, stable
    send_counts: list   # pairs this rank sends to each rank
    recv_counts: list   # pairs this rank receives from each rank
    experts_sorted: Any  # (P,) global expert ids in send order


def owner_of(expert_ids: Any, experts_per_rank: int) -> Any:
    return torch.div(expert_ids, experts_per_rank, rounding_mode="floor")


def plan_dispatch(top_i: Any, *, experts: int, world: int, group: Any = None) -> DispatchPlan:
    """``top_i (T, K)`` int64 global expert ids of the local tokens.  One count exchange (host-visible)."""
    import torch.distributed as dist

    if experts % world != 0:
        raise ValueError("experts=%d must divide evenly over %d ranks" % (experts, world))
    epr = experts // world
    flat = top_i.reshape(-1)
    if not flat.is_cuda and flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= experts):
        raise ValueError("expert id out of range")  # (device tensors come from the routing kernel, which cannot produce one)
    order = torch.argsort(flat, stable=True)
    experts_sorted = flat[order]
    send = torch.bincount(owner_of(experts_sorted, epr), minlength=world).to(torch.int64)
    if world == 1:
        return DispatchPlan(order, [int(send[0])], [int(send[0])], experts_sorted)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return DispatchPlan(order, [int(v) for v in send.tolist()], [int(v) for v in recv.tolist()], experts_sorted)


def all_to_all_rows(rows: Any, send_counts: list, recv_counts: list, *, world: int, group: Any = None) -> Any:
    """Variable-count all-to-all of the rows of ``rows`` (first dimension split by ``send_counts``)."""
    import torch.distributed as dist

    if world == 1:
        return rows
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out


def expert_parallel_moe(h: Any, top_w: Any, top_i: Any, *, experts: int, world: int, rank: int,
                        expert_fn: Callable[[Any, Any], Any], group: Any = None, section: Any = None) -> Any:
    """``h (T, H)`` fp16 normalised activations, ``top_w/top_i (T, K)``.  ``expert_fn(x (R, H), local_ids (R,))
    -> (R, H)`` fp16 runs this rank's experts on the received pairs.  Returns the fp32-combined, fp16-rounded
    MoE output ``(T, H)`` of the local tokens."""
    t, k = int(top_i.shape[0]), int(top_i.shape[1])
    epr = experts // world
    plan = plan_dispatch(top_i, experts=experts, world=world, group=group)
    send_x = h[torch.div(plan.order, k, rounding_mode="floor")]
    recv_x = all_to_all_rows(send_x, plan.send_counts, plan.recv_counts, world=world, group=group)
    recv_e = all_to_all_rows(plan.experts_sorted, plan.send_counts, plan.recv_counts, world=world, group=group)
    local_ids = recv_e - rank * epr
    if recv_x.shape[0]:
        # pairs arrive grouped by source rank; regroup by expert so each resident expert is streamed once
        perm = torch.argsort(local_ids, stable=True)
        y_sorted = expert_fn(recv_x[perm].contiguous(), local_ids[perm].contiguous())
        y = torch.empty_like(y_sorted)
        y[perm] = y_sorted
    else:
        y = recv_x.new_empty((0, h.shape[1]))
    back = all_to_all_rows(y, plan.recv_counts, plan.send_counts, world=world, group=group)
    pairs = torch.empty_like(back)
    pairs[plan.order] = back  # back to (t, k) order
    out = (pairs.reshape(t, k, -1).float() * top_w.reshape(t, k, 1).float()).sum(dim=1)
    return out.to(h.dtype)


class _NoSection:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _no_section(name: str) -> Any:
    return _NoSection()


ID_COLS = 8  # fp16 columns appended to a dispatched row (the first holds the expert id; 8 keep rows 16-byte aligned)


def expert_parallel_moe_static(h: Any, top_w: Any, top_i: Any, *, experts: int, world: int, rank: int,
                               expert_fn: Callable[[Any, Any], Any], group: Any = None, section: Any = _no_section) -> Any:
    """The same exchange with a STATIC capacity: every rank sends every peer a buffer of T*K pair slots (the
    worst case), unused slots carry the expert id ``experts`` and are sorted behind the real pairs, where
    ``expert_fn`` must ignore them.  The expert id rides in the row itself (one extra fp16 column group: ids up to
    2048 are exact in fp16), so a layer needs two all-to-alls: rows out, rows back.  No tensor shape and no
    collective size depends on the routing and nothing is read on the host, so the whole step can be captured in a
    CUDA graph.  Same results as :func:`expert_parallel_moe` bit for bit: every real pair meets the same kernel with
    the same inputs.  ``section(name)`` returns a context manager (timing hooks of the benchmark)."""
    import torch.distributed as dist

    if experts > 2048:
        raise ValueError("experts=%d: the id column of the static exchange is fp16 (exact up to 2048)" % experts)
    t, k = int(top_i.shape[0]), int(top_i.shape[1])
    pairs_n, hidden, epr, dev = t * k, int(h.shape[1]), experts // world, h.device
    with section("dispatch-combine glue"):
        flat = top_i.reshape(-1)
        order = torch.argsort(flat, stable=True)
        sorted_e = flat[order]
        dest = torch.div(sorted_e, epr, rounding_mode="floor")
        counts = (dest.reshape(-1, 1) == torch.arange(world, device=dev).reshape(1, -1)).sum(dim=0)
        starts = torch.cumsum(counts, dim=0) - counts
        pos = torch.arange(pairs_n, device=dev) - starts[dest]
        send = h.new_zeros((world, pairs_n, hidden + ID_COLS))
        send[:, :, hidden] = float(experts)
        send[dest, pos, :hidden] = h[torch.div(order, k, rounding_mode="floor")]
        send[dest, pos, hidden] = sorted_e.to(h.dtype)
    if world > 1:
        with section("all-to-all"):
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=group)
    else:
        recv = send
    with section("dispatch-combine glue"):
        recv_e = recv[:, :, hidden].reshape(-1).to(torch.int64)
        local = torch.where(recv_e == experts, torch.full_like(recv_e, epr), recv_e - rank * epr)
        perm = torch.argsort(local, stable=True)
        x_sorted = recv.reshape(-1, hidden + ID_COLS)[perm, :hidden].contiguous()
        ids_sorted = local[perm].contiguous()
    with section("expert kernels"):
        y_sorted = expert_fn(x_sorted, ids_sorted)
    with section("dispatch-combine glue"):
        y = torch.empty_like(y_sorted)
        y[perm] = y_sorted
        y = y.reshape(world, pairs_n, hidden)
    if world > 1:
        with section("all-to-all"):
            back = torch.empty_like(y)
            dist.all_to_all_single(back, y, group=group)
    else:
        back = y
    with section("dispatch-combine glue"):
        pairs = torch.empty((pairs_n, hidden), dtype=h.dtype, device=dev)
        pairs[order] = back[dest, pos]
        out = (pairs.reshape(t, k, -1).float() * top_w.reshape(t, k, 1).float()).sum(dim=1)
        return out.to(h.dtype)


def expert_parallel_moe_kernels(h: Any, top_w: Any, top_i: Any, *, experts: int, world: int, rank: int,
                                expert_fn: Callable[..., Any], group: Any = None, err_flag: Any = None,
                                section: Any = _no_section) -> Any:
    """:func:`expert_parallel_moe_static` for CUDA tensors with the row bookkeeping done by the library's exchange
    kernels (``lemoq_ep_*``): two launches to fill the send slots, two to regroup what arrived by local expert (which
    also yields the segment offsets of the expert kernels), one to give the results back, one for the weighted sum -
    where the tensor-library form needs some forty.  Same placement of every row, same collectives, so the two forms
    are interchangeable between ranks; the weighted sum is taken in slot order in fp32.  ``expert_fn(x_sorted, None,
    seg_offsets=seg)`` runs this rank's experts on rows in local-expert order."""
    import torch.distributed as dist

    from lemoq import _cabi

    if experts > 2048:
        raise ValueError("experts=%d: the id column of the static exchange is fp16 (exact up to 2048)" % experts)
    _cabi.require_cuda(h, top_w, top_i, what="expert-parallel exchange kernels")
    t, k = int(top_i.shape[0]), int(top_i.shape[1])
    pairs_n, hidden, epr, dev = t * k, int(h.shape[1]), experts // world, h.device
    rows = world * pairs_n
    stream = _cabi.current_stream(dev)
    err = _cabi.ptr(err_flag) if err_flag is not None else None
    h, top_i = h.contiguous(), top_i.contiguous()
    weights = top_w.to(torch.float16).contiguous()
    with section("dispatch-combine glue"):
        send = torch.empty((world, pairs_n, hidden + ID_COLS), dtype=torch.float16, device=dev)
        slot = torch.empty(pairs_n, dtype=torch.int32, device=dev)
        src = torch.empty(rows, dtype=torch.int32, device=dev)
        _cabi.call("lemoq_ep_dispatch", _cabi.ptr(h), _cabi.ptr(top_i), t, k, hidden, experts, world, _cabi.ptr(send), _cabi.ptr(slot),
                   _cabi.ptr(src), err, stream)
    if world > 1:
        with section("all-to-all"):
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=group)
    else:
        recv = send
    with section("dispatch-combine glue"):
        x_sorted = torch.empty((rows, hidden), dtype=torch.float16, device=dev)
        perm = torch.empty(rows, dtype=torch.int32, device=dev)
        seg = torch.empty(epr + 1, dtype=torch.int32, device=dev)
        _cabi.call("lemoq_ep_regroup", _cabi.ptr(recv), rows, hidden, experts, world, rank, _cabi.ptr(x_sorted), _cabi.ptr(perm),
                   _cabi.ptr(seg), err, stream)
    with section("expert kernels"):
        y_sorted = expert_fn(x_sorted, None, seg_offsets=seg)
    with section("dispatch-combine glue"):
        y = torch.empty((world, pairs_n, hidden), dtype=torch.float16, device=dev)
        _cabi.call("lemoq_ep_return", _cabi.ptr(y_sorted), _cabi.ptr(perm), _cabi.ptr(seg), rows, hidden, epr, _cabi.ptr(y), stream)
    if world > 1:
        with section("all-to-all"):
            back = torch.empty_like(y)
            dist.all_to_all_single(back, y, group=group)
    else:
        back = y
    with section("dispatch-combine glue"):
        out = torch.empty((t, hidden), dtype=torch.float16, device=dev)
        _cabi.call("lemoq_ep_combine", _cabi.ptr(back), _cabi.ptr(slot), _cabi.ptr(weights), t, k, hidden, _cabi.ptr(out), stream)
        return out.to(h.dtype)


# ---------------------------------------------------------------------------------------------------
# the CUDA side: this rank's experts and the batched lockstep decode step
# ---------------------------------------------------------------------------------------------------
class LocalExperts:
    """The W8 experts one rank owns in one layer; runs them through the grouped expert kernels."""

    def __init__(self, q: Any, lo: int, hi: int) -> None:
        self.gate_up = q.packed_gate_up[lo:hi].contiguous()
        self.gate_up_scale = q.scale_gate_up[lo:hi].contiguous()
        self.down = q.packed_down[lo:hi].contiguous()
        self.down_scale = q.scale_down[lo:hi].contiguous()
        self.group_size = int(q.group_size)
        self.n = hi - lo
        hidden, ffn = int(self.gate_up.shape[2]), int(self.down.shape[2])
        self.batched = hidden % 128 == 0 and hidden <= 4096 and ffn % 128 == 0 and ffn <= 4096 and self.group_size % 128 == 0

    def __call__(self, x: Any, local_ids: Any, seg_offsets: Any = None) -> Any:
        """``x (R, H)`` rows in local-expert order with either their ``local_ids (R,)`` or the ``seg_offsets`` of the
        experts' segments (the exchange kernels hand these over); returns the unweighted expert outputs ``(R, H)``."""
        from lemoq import _cabi
        from lemoq.kernels.batched_w8 import w8_experts_tokens

        _cabi.require_cuda(x, what="expert-parallel decode")
        if self.batched:
            # weights-stationary kernels: every resident expert's rows are read once for all its pairs
            return w8_experts_tokens(x, local_ids, self.gate_up, self.gate_up_scale, self.down, self.down_scale,
                                     group_size=self.group_size, seg_offsets=seg_offsets)
        if local_ids is None:
            raise NotImplementedError("expert shapes outside the many-token kernels need the row ids (use the tensor-library exchange)")
        r, hidden = int(x.shape[0]), int(x.shape[1])
        ffn = int(self.down.shape[2])
        ids = local_ids.to(torch.int64).reshape(r, 1).contiguous()
        ones = torch.ones((r, 1), dtype=torch.float16, device=x.device)
        act = torch.empty((r, 1, ffn), dtype=torch.float16, device=x.device)
        out = torch.empty((r, hidden), dtype=torch.float16, device=x.device)
        stream = _cabi.current_stream(x.device)
        _cabi.call("lemoq_moe_gate_up_w8", _cabi.ptr(x), _cabi.ptr(self.gate_up), _cabi.ptr(self.gate_up_scale), _cabi.ptr(ids),
                   r, 1, self.n, hidden, ffn, self.group_size, _cabi.ptr(act), None, stream)
        _cabi.call("lemoq_moe_down_w8", _cabi.ptr(act), _cabi.ptr(self.down), _cabi.ptr(self.down_scale), _cabi.ptr(ids),
                   _cabi.ptr(ones), r, 1, self.n, hidden, ffn, self.group_size, _cabi.ptr(out), None, stream)
        return out


class ExpertParallelDecoder:
    """Lockstep greedy decode of ``sequences`` sequences that share one prefilled prompt.

    ``model`` is the canonical quantised module tree (after ``install_replacements``); ``session`` a batch-1
    ``StaticCacheDecodeSession`` on it whose prefill filled the fp16 cache for the common prompt."""

    def __init__(self, model: Any, session: Any, *, sequences: int, world: int, rank: int, group: Any = None,
                 attn_splits: int = 4, static_exchange: bool = False, exchange_kernels: bool = True) -> None:
        from lemoq import _cabi

        if sequences % world != 0:
            raise ValueError("sequences=%d must divide evenly over %d ranks" % (sequences, world))
        cfg = model.config
        if cfg.num_experts % world != 0:
            raise ValueError("experts=%d must divide evenly over %d ranks" % (cfg.num_experts, world))
        self.model, self.cfg, self.world, self.rank, self.group = model, cfg, world, rank, group
        self.b = sequences // world
        self.first_seq = rank * self.b
        self.device = model.lm_head.packed.device
        self.heads, self.dim, self.hidden = cfg.num_attention_heads, cfg.head_dim, cfg.hidden_size
        self.max_len = int(session.config.max_cache_len)
        self.position = int(session.position)
        self.splits = attn_splits
        self.static_exchange = static_exchange
        # the static exchange with the library's row kernels (default) or written with tensor-library calls
        self.exchange_kernels = bool(exchange_kernels and static_exchange)
        self.graph = None
        epr = cfg.num_experts // world
        self.local = [LocalExperts(layer.mlp._static_experts, rank * epr, (rank + 1) * epr) for layer in model.model.layers]
        if static_exchange and not all(le.batched for le in self.local):
            raise NotImplementedError("the static-capacity exchange needs the many-token expert kernels (widths % 512 == 0, <= 2048)")
        self.cos, self.sin = model.model.rotary_emb.tables(self.max_len, torch.float16, self.device)
        # int8 KV of the shared prompt, replicated for the b local sequences: (b*heads, S, D) / (b*heads, S)
        self.kv = []
        stream = _cabi.current_stream(self.device)
        for i, _ in enumerate(model.model.layers):
            cl = session.cache.layers[i]
            _, h, s, d = (int(v) for v in cl.keys.shape)
            kc = torch.empty((h, s, d), dtype=torch.int8, device=self.device)
            vc = torch.empty_like(kc)
            ks = torch.empty((h, s), dtype=torch.float16, device=self.device)
            vs = torch.empty_like(ks)
            _cabi.call("lemoq_kv_int8_bulk_quantize", _cabi.ptr(cl.keys), _cabi.ptr(cl.values), _cabi.ptr(kc), _cabi.ptr(ks),
                       _cabi.ptr(vc), _cabi.ptr(vs), h, s, d, self.position, stream)
            self.kv.append({"kc": kc.repeat(self.b, 1, 1).contiguous(), "vc": vc.repeat(self.b, 1, 1).contiguous(),
                            "ks": ks.repeat(self.b, 1).contiguous(), "vs": vs.repeat(self.b, 1).contiguous()})
        ws_bytes = int(_cabi.lib().lemoq_attn_workspace_bytes(self.b * self.heads, self.dim, self.splits))
        self.attn_ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=self.device)
        self.pos_t = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.filled_t = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sections = None  # name -> list of (start, end) CUDA events while a timing split is being taken

    def _section(self, name: str) -> Any:
        if self.sections is None:
            return _NoSection()
        dec = self

        class _Timed:
            def __enter__(self_inner):
                self_inner.start = torch.cuda.Event(enable_timing=True)
                self_inner.start.record()
                return self_inner

            def __exit__(self_inner, *exc):
                end = torch.cuda.Event(enable_timing=True)
                end.record()
                dec.sections.setdefault(name, []).append((self_inner.start, end))
                return False

        return _Timed()

    def timing_split(self, tokens: Any, steps: int = 3) -> dict:
        """Microseconds per step by category, from CUDA events around the sections of ``steps`` EAGER steps at the
        current position (the position does not advance; a captured graph cannot be split this way, so launch gaps of
        the eager glue are inside the figures)."""
        graph, self.graph = self.graph, None
        pos = self.position
        try:
            self._forward_at(tokens)  # warm
            self.sections = {}
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(steps):
                self._forward_at(tokens)
            t1.record()
            torch.cuda.synchronize(self.device)
            out = {name: sum(a.elapsed_time(b) for a, b in evs) * 1e3 / steps for name, evs in self.sections.items()}
            out["whole eager step"] = t0.elapsed_time(t1) * 1e3 / steps
        finally:
            self.sections = None
            self.graph = graph
            self.position = pos
        return {k: round(v, 1) for k, v in out.items()}

    def _forward_at(self, tokens: Any) -> Any:
        self.pos_t.fill_(self.position)
        self.filled_t.fill_(self.position + 1)
        return self._forward(tokens)

    # -- one lockstep step: tokens (b,) int64 -> logits (b, V) fp16 -------------------------------------
    def step(self, tokens: Any) -> Any:
        if self.position >= self.max_len:
            raise RuntimeError("decode position exceeded StaticCache capacity")
        self.pos_t.fill_(self.position)
        self.filled_t.fill_(self.position + 1)
        if self.graph is not None:
            self.static_tokens.copy_(tokens)
            self.graph.replay()
            out = self.static_logits
        else:
            out = self._forward(tokens)
        self.position += 1
        return out

    def capture(self, warmup: int = 2) -> None:
        """Capture the step (exchange included) in one CUDA graph; needs the static-capacity exchange.  The warm-up
        steps run eagerly at the current position and are undone (the position does not advance)."""
        if not self.static_exchange:
            raise RuntimeError("graph capture needs static_exchange=True (the dynamic exchange reads counts on the host)")
        self.static_tokens = torch.zeros(self.b, dtype=torch.int64, device=self.device)
        self.pos_t.fill_(self.position)
        self.filled_t.fill_(self.position + 1)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._forward(self.static_tokens)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        # thread_local: the process group's watchdog thread may call CUDA while this thread captures
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self.static_logits = self._forward(self.static_tokens)
        self.graph = graph

    def _forward(self, tokens: Any) -> Any:
        from lemoq import _cabi
        from lemoq.kernels.batched_w8 import w8_linear_tokens
        from lemoq.kernels.dequant_gemv import dequant_gemm_fused
        from lemoq.kernels.rmsnorm import rms_norm_fused

        def linear(xin, codes, scale, gs):
            # many tokens: the weights-stationary kernel; shapes it does not take go through the per-token GEMV
            k = int(codes.shape[1])
            if k % 128 == 0 and k <= 4096 and gs % 128 == 0 and int(codes.shape[0]) % 2 == 0:
                return w8_linear_tokens(xin, codes, scale, group_size=gs)
            return dequant_gemm_fused(xin, codes, scale, group_size=gs, out_dtype=torch.float16)
        from lemoq.kernels.routing import routing_softmax_topk

        cfg, b, heads, dim = self.cfg, self.b, self.heads, self.dim
        a = heads * dim
        stream = _cabi.current_stream(self.device)
        # the position lives in device scalars (pos_t / filled_t) so that a captured graph follows it
        cos_row = self.cos.index_select(0, self.pos_t).reshape(-1).contiguous()
        sin_row = self.sin.index_select(0, self.pos_t).reshape(-1).contiguous()
        moe_fn = expert_parallel_moe_static if self.static_exchange else expert_parallel_moe
        if self.exchange_kernels and all(le.batched for le in self.local):
            def moe_fn(*args, **kwargs):  # noqa: E306
                return expert_parallel_moe_kernels(*args, err_flag=self.err, **kwargs)
        x = self.model.model.embed_tokens.weight[tokens]  # (b, H) fp16
        eps = float(cfg.rms_norm_eps)
        sec = self._section
        for i, layer in enumerate(self.model.model.layers):
            attn, mlp = layer.self_attn, layer.mlp
            pk = attn._lemoq_packed_qkv
            gs = int(pk.group_size)
            dense = sec("dense + attention")
            dense.__enter__()
            h1 = rms_norm_fused(x, layer.input_layernorm.weight, eps)
            qkv = linear(h1, pk.packed, pk.scale, gs)  # (b, 3A)
            q = rms_norm_fused(qkv[:, :a].contiguous(), attn.q_norm.weight, eps)
            k = rms_norm_fused(qkv[:, a:2 * a].contiguous(), attn.k_norm.weight, eps)
            v = qkv[:, 2 * a:].contiguous()
            q_r, k_r = torch.empty_like(q), torch.empty_like(k)
            # batch x heads act as heads: every sequence is at the same position
            _cabi.call("lemoq_rope_qk", _cabi.ptr(q), dim, b * heads, _cabi.ptr(k), dim, b * heads, _cabi.ptr(cos_row),
                       _cabi.ptr(sin_row), dim, _cabi.ptr(q_r), _cabi.ptr(k_r), stream)
            kv = self.kv[i]
            _cabi.call("lemoq_kv_int8_cache_write", _cabi.ptr(k_r), _cabi.ptr(v), _cabi.ptr(kv["kc"]), _cabi.ptr(kv["ks"]),
                       _cabi.ptr(kv["vc"]), _cabi.ptr(kv["vs"]), _cabi.ptr(self.pos_t), b * heads, self.max_len, dim,
                       _cabi.ptr(self.err), stream)
            ctx_out = torch.empty((b, a), dtype=torch.float16, device=self.device)
            _cabi.call("lemoq_attn_decode_int8", _cabi.ptr(q_r), _cabi.ptr(kv["kc"]), _cabi.ptr(kv["ks"]), _cabi.ptr(kv["vc"]),
                       _cabi.ptr(kv["vs"]), self.max_len * dim, _cabi.ptr(self.filled_t), _cabi.ptr(ctx_out), b * heads,
                       self.max_len, dim, self.splits, 1.0 / math.sqrt(dim), _cabi.ptr(self.attn_ws), _cabi.ptr(self.err), stream)
            o = linear(ctx_out, attn.o_proj.packed, attn.o_proj.scale, gs)
            x1 = o + x
            h2 = rms_norm_fused(x1, layer.post_attention_layernorm.weight, eps)
            logits = torch.matmul(h2, mlp._static_router.t())  # (b, E) fp16: a plain library GEMM
            top_w, top_i = routing_softmax_topk(logits, top_k=cfg.num_experts_per_tok, norm_topk_prob=bool(cfg.norm_topk_prob))
            dense.__exit__(None, None, None)
            moe = moe_fn(h2, top_w.to(torch.float16), top_i, experts=cfg.num_experts, world=self.world,
                         rank=self.rank, expert_fn=self.local[i], group=self.group, section=sec)
            x = moe + x1
        with sec("dense + attention"):
            hn = rms_norm_fused(x, self.model.model.norm.weight, eps)
            lm = self.model.lm_head
            return linear(hn, lm.packed, lm.scale, int(lm.group_size))

    def error_flags(self) -> int:
        return int(self.err.item())


def token_digest(hist: Any) -> str:
    """Digest of a (sequences, steps) int64 token table (little-endian bytes, SHA-256)."""
    import hashlib

    return hashlib.sha256(hist.to(torch.int64).cpu().contiguous().numpy().tobytes()).hexdigest()


def measure(model: Any, *, device: str, world: int, rank: int, sequences: int = 64, ctx: int = 2048, steps: int = 32,
            warmup: int = 3, exchange: str = "static", graph: bool = True, identical: bool = False, split: bool = True,
            attn_splits: int | None = None) -> dict:
    """Prefill the shared prompt, build this rank's share of the lockstep decoder, decode ``warmup + steps`` tokens
    per sequence and time the last ``steps`` (device events, max over ranks).  ``model`` is the canonical quantised
    module tree.  Returns the result record (every rank; token table and digest are those of all sequences)."""
    import gc

    import torch.distributed as dist

    from benchmarks.cudagraph import StaticCacheDecodeSession

    horizon = steps + warmup + 2
    prompt = torch.full((1, ctx), 1, dtype=torch.long, device=device)
    session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=horizon, device=device, engine="ops")  # prefills
    extra = {} if attn_splits is None else {"attn_splits": int(attn_splits)}
    dec = ExpertParallelDecoder(model, session, sequences=sequences, world=world, rank=rank, static_exchange=exchange == "static", **extra)
    if graph:
        dec.capture()
    # the literal configuration decodes identical sequences; distinct first tokens make the exchange non-trivial
    first = torch.arange(dec.first_seq, dec.first_seq + dec.b, device=device, dtype=torch.int64)
    tokens = (first * 7 + 2) % model.config.vocab_size if not identical else torch.full_like(first, int(session.seed_token_id))
    history = []

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(warmup):
        tokens = dec.step(tokens).float().argmax(dim=-1)
        history.append(tokens.clone())
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        tokens = dec.step(tokens).float().argmax(dim=-1)
        history.append(tokens.clone())
    e1.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    ms = torch.tensor([max(e0.elapsed_time(e1), wall_ms)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    hist = torch.stack(history, dim=1)  # (b, warmup + steps)
    if world > 1:
        gathered = [torch.empty_like(hist) for _ in range(world)]
        dist.all_gather(gathered, hist)
        hist = torch.cat(gathered, dim=0)
    parts = dec.timing_split(tokens) if split else None
    flags = dec.error_flags()
    alone_ms = None
    if world > 1 and graph and exchange == "static":
        alone_ms = _collectives_alone_ms(dec, model.config, world, device, barrier)
    # a captured graph holds collective kernels of the process group: destroy it (not only drop the name) before
    # anybody tears the communicator down, whose shutdown waits for every captured plan to be released
    if dec.graph is not None:
        dec.graph.reset()
        dec.graph = None
    session.close()
    del dec, session
    gc.collect()
    torch.cuda.synchronize()
    ms_step = float(ms.item()) / steps
    cfg = model.config
    return {"metric": "decode_tokens_per_s_batched_expert_parallel", "value": sequences * 1000.0 / ms_step, "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "data": "synthetic",
            "config": {"workload": "%d sequences x ctx %d lockstep greedy decode, W8A16 + INT8 KV, experts sharded %d per GPU, "
                                   "NCCL all-to-all dispatch/combine (benchmark configuration 5)" % (sequences, ctx, cfg.num_experts // world),
                       "layers": cfg.num_hidden_layers, "identical_sequences": bool(identical), "exchange": exchange,
                       "cuda_graph": bool(graph), "all_to_alls_per_step": 2 * cfg.num_hidden_layers if world > 1 else 0},
            "eager_split_us_per_step": parts, "all_to_alls_alone_ms_per_step": alone_ms, "error_flags": flags,
            "token_digest": token_digest(hist), "tokens": hist.cpu()}


def _collectives_alone_ms(dec: Any, cfg: Any, world: int, device: str, barrier: Callable[[], None], iters: int = 5) -> float:
    """Device time of the all-to-alls of one step ALONE, in a CUDA graph of their own: same buffers shapes, same count
    (two per layer), nothing in between.  What the step cannot get below at this world size.  Max over ranks."""
    import torch.distributed as dist

    pairs = dec.b * int(cfg.num_experts_per_tok)
    hidden = int(cfg.hidden_size)
    send = torch.zeros((world, pairs, hidden + ID_COLS), dtype=torch.float16, device=device)
    recv = torch.empty_like(send)
    y = torch.zeros((world, pairs, hidden), dtype=torch.float16, device=device)
    back = torch.empty_like(y)

    def exchanges():
        for _ in range(int(cfg.num_hidden_layers)):
            dist.all_to_all_single(recv, send, group=dec.group)
            dist.all_to_all_single(back, y, group=dec.group)

    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        exchanges()
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        exchanges()
    g.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=device, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    g.reset()  # before anybody tears the communicator down (see measure())
    del g
    return float(ms.item())


def shutdown_process_group(limit_s: float = 60.0) -> None:
    """``destroy_process_group`` with a host-side time limit.  The communicator's shutdown waits until every CUDA graph
    that captured one of its collectives has been destroyed; :func:`measure` destroys its graph first.  Should the
    shutdown still not return within ``limit_s`` the process leaves without it (all results are out by then)."""
    import threading

    import torch.distributed as dist

    def give_up():
        sys.stderr.write("expert_parallel: process-group shutdown did not return within %.0f s; leaving without it\n" % limit_s)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    timer = threading.Timer(limit_s, give_up)
    timer.daemon = True
    timer.start()
    dist.destroy_process_group()
    timer.cancel()


def run(args: Any) -> int:
    import torch.distributed as dist

    from benchmarks.runner import build_model, install_replacements

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = "cuda:%d" % local_rank
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    model = build_model(seed=0, device=device, layers=args.layers)
    install_replacements(model, attn="kernel", moe="grouped", quant_cfg={"bit_width": "w8a16", "dequant": "fused", "group_size": 128},
                         rmsnorm="fused", ctx=args.ctx, max_new_tokens=args.steps + args.warmup + 2, device=device)
    result = measure(model, device=device, world=world, rank=rank, sequences=args.sequences, ctx=args.ctx, steps=args.steps,
                     warmup=args.warmup, exchange=args.exchange, graph=args.graph, identical=args.identical, attn_splits=args.attn_splits)
    hist = result.pop("tokens")
    if rank == 0:
        if args.check_against:
            ref = torch.load(args.check_against)
            result["tokens_match_reference_run"] = bool(tuple(ref.shape) == tuple(hist.shape) and torch.equal(ref, hist))
        print(json.dumps(result))
        if args.tokens_out:
            torch.save(hist, args.tokens_out)
    if world > 1:
        dist.barrier()
        shutdown_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sequences", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None, help="decode a model of this many layers instead of 16")
    ap.add_argument("--exchange", default="static", choices=["static", "dynamic"],
                    help="static: fixed-capacity all-to-all, nothing read on the host; dynamic: counts exchanged and read per layer")
    ap.add_argument("--graph", action="store_true", help="capture the step (with its all-to-alls) in one CUDA graph; static exchange only")
    ap.add_argument("--attn-splits", type=int, default=None, help="splits of the key range per (sequence, head) in the attention kernel")
    ap.add_argument("--identical", action="store_true", help="all sequences start from the prompt's own next token")
    ap.add_argument("--tokens-out", default=None, help="rank 0 saves the (sequences, warmup+steps) decoded tokens here")
    ap.add_argument("--check-against", default=None, help="a --tokens-out file of another world size: must match token for token")
    return run(ap.parse_args())


if __name__ == "__main__":
    raise SystemExit(main())
