"""CPU restatement of the LeanMoE-Quant batch-1 decode arithmetic.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path: it is
imported by the test-suite, by the smoke check and by the CPU-baseline leg of
the benchmark, never by the product package.  Every function states the
reference file:line it follows (paths are relative to the reference project).

Parity status: PINNED.  ``tests/golden/`` holds vectors produced by importing
the reference's own Python functions (``tests/golden/make_golden.py``) and
``tests/test_oracle_golden.py`` checks every function here against them.

All arithmetic is plain torch on CPU tensors.  Rounding points are explicit:
``.half()`` marks every place where the reference rounds to fp16.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

LOG2E = 1.4426950408889634  # src/lemoq/kernels/attn_decode.py:104
KV_QMAX = 127.0  # src/lemoq/kernels/kv_int8.py:27


# --------------------------------------------------------------------------
# weight quantisation: per-row, per-group symmetric round-to-nearest
# --------------------------------------------------------------------------
def rtn_quantize_w8(weight: torch.Tensor, group_size: int = 128):
    """8-bit symmetric RTN along the last dim, one scale per (row, group).

    Follows src/lemoq/quant/rtn.py:38-99 (symmetric branch) as used by
    src/lemoq/kernels/moe_grouped_quant.py:191-244 and src/lemoq/quant/linear.py:275-321:
    fp32 ``absmax/127`` scale (1.0 for an all-zero group), ``round(w/scale)``
    half-to-even computed with the fp32 scale, clamp to [-128, 127]; the scale is
    stored as fp16 only after the codes exist.

    Returns ``(codes int8 (..., in), scale fp16 (..., in/group))``.  The input
    width must be a multiple of ``group_size`` (the decode kernels carry no K
    mask: src/lemoq/kernels/moe_grouped_quant.py:209-219).
    """
    if weight.shape[-1] % group_size != 0:
        raise ValueError("in_features %d not divisible by group_size %d" % (weight.shape[-1], group_size))
    lead = weight.shape[:-1]
    in_features = weight.shape[-1]
    groups = in_features // group_size
    w = weight.float().reshape(-1, groups, group_size)
    absmax = w.abs().amax(dim=2, keepdim=True)
    scale = torch.where(absmax > 0, absmax / 127.0, torch.ones_like(absmax))
    codes = (w / scale).round().clamp(-128, 127)
    return (
        codes.to(torch.int8).reshape(*lead, in_features),
        scale.reshape(*lead, groups).half(),
    )


def dequantize_w8(codes: torch.Tensor, scale: torch.Tensor, group_size: int = 128, dtype=torch.float32):
    """``codes * scale`` with the fp16 scale widened to fp32.

    Follows src/lemoq/kernels/moe_grouped_quant.py:152-163 and
    src/lemoq/quant/linear.py:365-395.
    """
    lead = codes.shape[:-1]
    in_features = codes.shape[-1]
    groups = in_features // group_size
    c = codes.float().reshape(*lead, groups, group_size)
    w = (c * scale.float().unsqueeze(-1)).reshape(*lead, in_features)
    return w.to(dtype)


# --------------------------------------------------------------------------
# dense W8 GEMV (q/k/v/o projections, lm_head)
# --------------------------------------------------------------------------
def dense_w8_gemv(x: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor, group_size: int = 128,
                  acc_dtype=torch.float32, out_dtype=torch.float16):
    """``y[m, n] = sum_k x[m, k] * codes[n, k] * scale[n, k // g]``.

    Follows src/lemoq/kernels/reference.py:47-58 (materialise then matmul) which is
    the oracle of src/lemoq/kernels/_dequant_triton.py:313-463; accumulate in
    ``acc_dtype``, round once to ``out_dtype``.
    """
    w = dequantize_w8(codes, scale, group_size, dtype=acc_dtype)
    y = x.to(acc_dtype) @ w.t()
    return y.to(out_dtype) if out_dtype is not None else y


# --------------------------------------------------------------------------
# RMSNorm and RoPE
# --------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5):
    """HF OlmoeRMSNorm semantics: normalise in fp32, round to the input dtype,
    then multiply by the weight in that dtype.

    Follows src/lemoq/kernels/rmsnorm.py:186-202 and the formula pinned at
    tests/test_rmsnorm_parity.py:20-26.
    """
    dt = x.dtype
    h = x.float()
    var = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(var + eps)
    return weight.to(dt) * h.to(dt)


def rope_tables(max_len: int, head_dim: int, theta: float = 10000.0, dtype=torch.float16):
    """cos/sin tables ``(max_len, head_dim)`` in the half-split layout.

    Restates HF ``OlmoeRotaryEmbedding`` (transformers 4.57.6, the dependency the
    reference pins in pyproject.toml:30 and calls at
    src/lemoq/kernels/attn_decode.py:917-926): ``inv_freq = theta^(-2i/D)``,
    ``angle = pos * inv_freq`` in fp32, ``cos/sin`` of ``[angle, angle]`` rounded
    to the model dtype.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    pos = torch.arange(max_len, dtype=torch.float32)
    freqs = pos[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """``out = x*cos + rotate_half(x)*sin`` in fp32, one rounding to x.dtype.

    ``x`` is ``(..., D)``; ``cos``/``sin`` broadcast over the leading dims.
    Follows src/lemoq/kernels/rope.py:101-123 (oracle: tests/test_fused_rope.py:121-126).
    """
    d = x.shape[-1]
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    rot = torch.cat((-x2, x1), dim=-1)
    return (xf * cos.float() + rot * sin.float()).to(x.dtype)


# --------------------------------------------------------------------------
# KV cache: per-token symmetric int8
# --------------------------------------------------------------------------
def kv_quantize_per_token(x: torch.Tensor):
    """Per-(head, token) symmetric int8 over the last dim.

    Follows src/lemoq/kernels/kv_int8.py:30-41: fp32 ``amax/127`` (1.0 for a zero
    row), true division ``x/s``, round half-to-even, clamp to +-127, scale stored
    as fp16.  Returns ``(codes int8 (..., D), scale fp16 (...,))``.
    """
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / KV_QMAX, torch.ones_like(amax))
    q = torch.round(xf / scale).clamp_(-127, 127)
    return q.to(torch.int8), scale.half().squeeze(-1)


def kv_bulk_quantize(keys: torch.Tensor, values: torch.Tensor, filled: Optional[int] = None):
    """Quantise a whole fp16 cache ``(1, H, S, D)`` into the int8 mirror.

    Follows src/lemoq/kernels/kv_int8.py:127-163: slots at or beyond ``filled``
    hold code 0 / scale 1; ``filled=None`` quantises every slot (a zero row also
    yields code 0 / scale 1).  ``filled <= 0`` takes the same branch as ``None``
    there (the test is ``filled is not None and filled > 0``, :147), so it
    quantises every slot too.
    """
    _, h, s, d = keys.shape
    out = {}
    for name, t in (("k", keys), ("v", values)):
        codes = torch.zeros((1, h, s, d), dtype=torch.int8)
        scales = torch.ones((1, h, s), dtype=torch.float16)
        n = s if filled is None or int(filled) <= 0 else min(int(filled), s)
        if n > 0:
            c, sc = kv_quantize_per_token(t[0, :, :n, :])
            codes[0, :, :n, :] = c
            scales[0, :, :n] = sc
        out[name + "c"] = codes
        out[name + "s"] = scales
    return out


def kv_slot_write(cache: torch.Tensor, pos: int, row: torch.Tensor):
    """Bit copy of a ``(1, H, 1, D)`` row into ``cache[:, :, pos]``, touching no
    other slot.  Follows src/lemoq/kernels/kv_write.py:28-50 and
    src/lemoq/kernels/kv_direct.py:78-104."""
    cache[:, :, pos: pos + 1, :] = row
    return cache


# --------------------------------------------------------------------------
# decode attention
# --------------------------------------------------------------------------
def attention_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, filled: int,
                    scale: Optional[float] = None, dtype=torch.float64):
    """softmax(q k^T * scale) v over positions ``[0, filled)``; ``filled == 0`` gives
    zeros.  ``q`` is ``(H, D)``, ``k``/``v`` are ``(H, S, D)``.

    Follows src/lemoq/kernels/attn_decode.py:383-413 (``dense_attention_oracle``).
    """
    h, d = q.shape
    n = int(filled)
    if n == 0:
        return torch.zeros((h, d), dtype=dtype)
    scale = (1.0 / math.sqrt(d)) if scale is None else float(scale)
    qq = q.to(dtype)
    kk = k[:, :n, :].to(dtype)
    vv = v[:, :n, :].to(dtype)
    scores = torch.matmul(kk, qq.unsqueeze(-1)).squeeze(-1) * scale
    w = torch.softmax(scores, dim=-1)
    return torch.matmul(w.unsqueeze(1), vv).squeeze(1)


def attention_int8(q: torch.Tensor, kc: torch.Tensor, ks: torch.Tensor, vc: torch.Tensor,
                   vs: torch.Tensor, filled: int, scale: Optional[float] = None, dtype=torch.float64):
    """Dequantise the int8 mirror then run dense attention.

    ``q (H, D)``; ``kc``/``vc`` ``(H, S, D)`` int8; ``ks``/``vs`` ``(H, S)`` fp16.
    Follows the gate oracle at tests/test_kv_int8_read_gpu.py:69-86; the kernel's
    folded form (src/lemoq/kernels/_attn_triton.py:102-165) is algebraically
    identical.
    """
    k_true = kc.to(dtype) * ks.to(dtype).unsqueeze(-1)
    v_true = vc.to(dtype) * vs.to(dtype).unsqueeze(-1)
    return attention_dense(q, k_true, v_true, filled, scale=scale, dtype=dtype)


def attention_split_kv(q, k, v, filled: int, num_splits: int, block_n: int = 128,
                       scale: Optional[float] = None):
    """Split-KV online softmax (base 2) followed by the fixed-order LSE merge, fp32.

    Follows src/lemoq/kernels/attn_decode.py:295-380: split ``s`` covers
    ``[s*ceil(n/NS), ...)``; an empty split contributes ``(m=-inf, l=0, acc=0)``;
    all-empty merges to 0, not NaN.
    """
    h, d = q.shape
    n = int(filled)
    scale = (1.0 / math.sqrt(d)) if scale is None else float(scale)
    qk_scale = scale * LOG2E
    qf, kf, vf = q.float(), k.float(), v.float()
    m = torch.full((h, num_splits), float("-inf"))
    l = torch.zeros((h, num_splits))
    acc = torch.zeros((h, num_splits, d))
    if n > 0:
        chunk = -(-n // num_splits)
        for s in range(num_splits):
            start, end = s * chunk, min(s * chunk + chunk, n)
            if start >= end:
                continue
            m_i = torch.full((h,), float("-inf"))
            l_i = torch.zeros((h,))
            a_i = torch.zeros((h, d))
            for n0 in range(start, end, block_n):
                hi = min(n0 + block_n, end)
                qk = torch.matmul(kf[:, n0:hi], qf.unsqueeze(-1)).squeeze(-1) * qk_scale
                m_new = torch.maximum(m_i, qk.max(dim=1).values)
                alpha = torch.exp2(m_i - m_new)
                p = torch.exp2(qk - m_new.unsqueeze(1))
                l_i = l_i * alpha + p.sum(dim=1)
                a_i = a_i * alpha.unsqueeze(1) + torch.matmul(p.unsqueeze(1), vf[:, n0:hi]).squeeze(1)
                m_i = m_new
            m[:, s], l[:, s], acc[:, s] = m_i, l_i, a_i
    big = m.max(dim=1, keepdim=True).values
    big = torch.where(torch.isfinite(big), big, torch.zeros_like(big))
    w = torch.exp2(m - big)
    num = (acc * w.unsqueeze(-1)).sum(dim=1)
    den = (l * w).sum(dim=1)
    safe = den.clamp_min(torch.finfo(torch.float32).tiny).unsqueeze(1)
    return torch.where(den.unsqueeze(1) > 0, num / safe, num)


# --------------------------------------------------------------------------
# routing and grouped experts
# --------------------------------------------------------------------------
def routing_softmax_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool = False):
    """fp32 softmax over experts, then ``top_k`` rounds of arg-max (lowest index
    wins a tie), optional renormalisation.

    Follows src/lemoq/kernels/_routing_triton.py:43-80 and the ATen arm at
    src/lemoq/kernels/moe_static.py:279-283 (stable descending order:
    tests/test_routing_fusion.py:24-35).  Returns ``(top_w fp32 (T,K), top_i int64 (T,K))``.
    """
    p = torch.softmax(logits.float(), dim=-1)
    t, e = p.shape
    top_w = torch.empty((t, top_k), dtype=torch.float32)
    top_i = torch.empty((t, top_k), dtype=torch.int64)
    cur = p.clone()
    rows = torch.arange(t)
    for k in range(top_k):
        mx = cur.max(dim=-1, keepdim=True).values
        idx = (cur == mx).to(torch.uint8).argmax(dim=-1)  # first maximal index
        top_i[:, k] = idx
        top_w[:, k] = p[rows, idx]
        cur[rows, idx] = -1.0e30
    if norm_topk_prob:
        top_w = top_w / top_w.sum(dim=-1, keepdim=True)
    return top_w, top_i


def route(x: torch.Tensor, router_weight: torch.Tensor, top_k: int, norm_topk_prob: bool = False):
    """Router: fp16 logits from an fp32-accumulated dot, softmax/top-k, weights
    cast back to the activation dtype.

    Follows src/lemoq/kernels/moe_static.py:262-283.  Returns
    ``(logits (T,E) x.dtype, top_w (T,K) x.dtype, top_i (T,K) int64)``.
    """
    logits = (x.float() @ router_weight.float().t()).to(x.dtype)
    top_w, top_i = routing_softmax_topk(logits, top_k, norm_topk_prob)
    return logits, top_w.to(x.dtype), top_i


def grouped_gate_up_act(x: torch.Tensor, gate_up: torch.Tensor, ids: torch.Tensor, ffn: int,
                        acc_dtype=torch.float32):
    """``act[i, n] = silu(Wg[e_i, n, :] . x) * (Wu[e_i, n, :] . x)``.

    ``x (H,)``, ``gate_up (E, 2F, H)`` dequantised weights (gate rows ``[0, F)``,
    up rows ``[F, 2F)``), ``ids (K,)``.  Follows
    src/lemoq/kernels/moe_grouped.py:147-183.  Returns ``(K, F)`` in ``acc_dtype``.
    """
    xf = x.reshape(-1).to(acc_dtype)
    w = gate_up[ids].to(acc_dtype)
    gate = w[:, :ffn, :] @ xf
    up = w[:, ffn:, :] @ xf
    return gate * torch.sigmoid(gate) * up


def grouped_down_sum(act: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, top_w: torch.Tensor,
                     acc_dtype=torch.float32):
    """``out[n] = sum_i top_w[i] * (Wd[e_i, n, :] . act[i, :])``.

    Follows src/lemoq/kernels/moe_grouped.py:186-206.  Returns ``(H,)``.
    """
    w = down[ids].to(acc_dtype)  # (K, H, F)
    y = torch.matmul(w, act.to(acc_dtype).unsqueeze(-1)).squeeze(-1)
    y = y * top_w.reshape(-1, 1).to(acc_dtype)
    return y.sum(dim=0)


@dataclass
class QuantExperts:
    """Stacked W8 experts.  Follows src/lemoq/kernels/moe_grouped_quant.py:72-100:
    ``gate_up`` codes ``(E, 2F, H)`` int8 + scale ``(E, 2F, H/g)`` fp16, ``down`` codes
    ``(E, H, F)`` int8 + scale ``(E, H, F/g)`` fp16."""

    packed_gate_up: torch.Tensor
    scale_gate_up: torch.Tensor
    packed_down: torch.Tensor
    scale_down: torch.Tensor
    group_size: int = 128

    @property
    def ffn(self) -> int:
        return int(self.packed_gate_up.shape[1]) // 2


def quantize_experts(gate_up: torch.Tensor, down: torch.Tensor, group_size: int = 128) -> QuantExperts:
    """RTN on the stacked tensors (row-local, so identical to per-expert RTN:
    src/lemoq/kernels/moe_grouped_quant.py:191-244)."""
    cg, sg = rtn_quantize_w8(gate_up, group_size)
    cd, sd = rtn_quantize_w8(down, group_size)
    return QuantExperts(cg.contiguous(), sg.contiguous(), cd.contiguous(), sd.contiguous(), group_size)


def grouped_moe_w8(x: torch.Tensor, q: QuantExperts, ids: torch.Tensor, top_w: torch.Tensor,
                   acc_dtype=torch.float32):
    """One-token grouped expert FFN on W8 weights: dequantise the selected experts,
    gate/up + SwiGLU rounded to fp16, down + weighted sum rounded to fp16.

    Follows src/lemoq/kernels/moe_grouped_quant.py:385-405,411-559 with
    ``backend="oracle"`` (``act`` and ``out`` are cast to the activation dtype at
    :478-480 and :523-526).  Only the ``K`` routed experts are dequantised; the
    arithmetic per expert is the same as dequantising all ``E``.
    """
    dt = x.dtype
    ids = ids.reshape(-1).long()
    g = q.group_size
    gu = dequantize_w8(q.packed_gate_up[ids], q.scale_gate_up[ids], g, dtype=acc_dtype)
    dn = dequantize_w8(q.packed_down[ids], q.scale_down[ids], g, dtype=acc_dtype)
    local = torch.arange(ids.numel())
    act = grouped_gate_up_act(x, gu, local, q.ffn, acc_dtype).to(dt)
    out = grouped_down_sum(act, dn, local, top_w.to(dt), acc_dtype).to(dt)
    return out, act


def grouped_moe_fp16(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor,
                     top_w: torch.Tensor, acc_dtype=torch.float32):
    """Same contract on unquantised fp16 expert weights
    (src/lemoq/kernels/moe_grouped.py:315-470 with ``backend="oracle"``)."""
    dt = x.dtype
    ids = ids.reshape(-1).long()
    ffn = int(gate_up.shape[1]) // 2
    act = grouped_gate_up_act(x, gate_up, ids, ffn, acc_dtype).to(dt)
    out = grouped_down_sum(act, down, ids, top_w.to(dt), acc_dtype).to(dt)
    return out, act


def moe_block_w8(h: torch.Tensor, router_weight: torch.Tensor, q: QuantExperts, top_k: int,
                 norm_topk_prob: bool = False):
    """Router + grouped experts for one token (src/lemoq/kernels/moe_grouped_quant.py:562-601).
    Returns ``(out (H,), logits (E,), top_w (K,), top_i (K,))``."""
    logits, top_w, top_i = route(h.reshape(1, -1), router_weight, top_k, norm_topk_prob)
    out, _ = grouped_moe_w8(h.reshape(-1), q, top_i.reshape(-1), top_w.reshape(-1))
    return out, logits.reshape(-1), top_w.reshape(-1), top_i.reshape(-1)


# --------------------------------------------------------------------------
# logits comparison gates
# --------------------------------------------------------------------------
def compare_logits(reference, candidate):
    """Mean over steps of ``KL(ref || got)`` in fp32 plus top-1 agreement.
    Follows benchmarks/cudagraph.py:298-325."""
    ref = torch.cat([x.detach().reshape(1, -1).float().cpu() for x in reference], dim=0)
    got = torch.cat([x.detach().reshape(1, -1).float().cpu() for x in candidate], dim=0)
    ref_logp = torch.log_softmax(ref, dim=-1)
    got_logp = torch.log_softmax(got, dim=-1)
    kl = (ref_logp.exp() * (ref_logp - got_logp)).sum(dim=-1).mean()
    agree = (ref.argmax(dim=-1) == got.argmax(dim=-1)).float().mean()
    return {"kl": max(float(kl), 0.0), "top1_agreement": float(agree)}
