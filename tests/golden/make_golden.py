"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available (it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/LeanMoE-Quant

Every array written here is the output of the reference's own Python function
(imported from ``<reference>/src``) or, for the pieces the reference delegates to
Hugging Face transformers, of the installed transformers' OLMoE modules.  Inputs are
seeded and stored beside the outputs, so the tests need neither the reference nor a
network.  Fixtures are small on purpose (a few hundred KB in total).
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return t.detach().cpu().numpy()


def gen_rtn(out):
    from lemoq.quant import rtn

    g = torch.Generator().manual_seed(11)
    w = torch.randn(24, 256, generator=g) * 0.02
    w[3, 128:] = 0.0  # an all-zero group -> scale 1.0, codes 0
    w[5, :128] = torch.linspace(-1, 1, 128)  # hits the +-127 ends exactly
    # values that land on .5 in code space (half-to-even)
    w[7, :128] = 0.0
    w[7, 0] = 127.0
    w[7, 1:9] = torch.tensor([0.5, 1.5, 2.5, 3.5, -0.5, -1.5, -2.5, 126.5])
    q = rtn.quantize_rtn(w, bits=8, group_size=128, symmetric=True)
    out["rtn_w"] = _np(w)
    out["rtn_codes"] = _np(q["codes"].to(torch.int8))
    out["rtn_scale_fp32"] = _np(q["scale"])
    out["rtn_scale_fp16"] = _np(q["scale"].half())


def gen_experts(out):
    from lemoq.kernels.moe_grouped_quant import (
        grouped_moe_forward_quant,
        quantize_fused_experts,
        static_moe_forward_grouped_quant,
    )
    from lemoq.kernels.moe_grouped import grouped_moe_forward
    from lemoq.kernels.moe_static import FusedExperts

    g = torch.Generator().manual_seed(12)
    e, f, h, k = 4, 128, 128, 2
    gate_up = (torch.randn(e, 2 * f, h, generator=g) * 0.05).half()
    down = (torch.randn(e, h, f, generator=g) * 0.05).half()
    fused = FusedExperts(gate_up=gate_up, down=down)
    q = quantize_fused_experts(fused, bits=8, group_size=128)
    x = torch.randn(h, generator=g).half()
    ids = torch.tensor([3, 1], dtype=torch.int64)
    top_w = torch.tensor([0.31, 0.12]).half()
    y = grouped_moe_forward_quant(x, q, ids, top_w, backend="oracle")
    y16 = grouped_moe_forward(x, fused, ids, top_w, backend="oracle")
    router = (torch.randn(e, h, generator=g) * 0.05).half()
    blk, logits = static_moe_forward_grouped_quant(
        x.reshape(1, 1, h), router, q, top_k=k, norm_topk_prob=False, act_fn=None, backend="oracle")
    out.update(
        moe_gate_up=_np(gate_up), moe_down=_np(down),
        moe_gu_codes=_np(q.packed_gate_up), moe_gu_scale=_np(q.scale_gate_up),
        moe_dn_codes=_np(q.packed_down), moe_dn_scale=_np(q.scale_down),
        moe_x=_np(x), moe_ids=_np(ids), moe_top_w=_np(top_w), moe_out_w8=_np(y), moe_out_fp16=_np(y16),
        moe_router=_np(router), moe_block_out=_np(blk.reshape(-1)), moe_block_logits=_np(logits.reshape(-1)),
    )


def gen_dense(out):
    from lemoq.kernels.reference import dequant_gemm_fused_reference, dequant_gemm_separate_reference
    from lemoq.quant import rtn

    g = torch.Generator().manual_seed(13)
    w = torch.randn(40, 384, generator=g) * 0.03
    q = rtn.quantize_rtn(w, bits=8, group_size=128, symmetric=True)
    codes = q["codes"].to(torch.int8)
    scale = q["scale"].half()
    x = torch.randn(2, 384, generator=g).half()
    y_sep = dequant_gemm_separate_reference(x, codes, scale, None, group_size=128)
    y_fus = dequant_gemm_fused_reference(x, codes, scale, None, group_size=128)
    out.update(dense_codes=_np(codes), dense_scale=_np(scale), dense_x=_np(x),
               dense_y_separate=_np(y_sep), dense_y_fused=_np(y_fus))


def gen_kv(out):
    from lemoq.kernels.kv_int8 import kv_int8_bulk_quantize, quantize_per_token_int8

    g = torch.Generator().manual_seed(14)
    row = torch.randn(1, 4, 1, 64, generator=g).half()
    row[0, 2] = 0.0  # zero row -> scale 1, codes 0
    row[0, 3, 0, :4] = torch.tensor([1.0, 0.5 / 127, 1.5 / 127, -2.5 / 127]).half()
    c, s = quantize_per_token_int8(row)
    cache_k = torch.randn(1, 4, 12, 64, generator=g).half()
    cache_v = torch.randn(1, 4, 12, 64, generator=g).half()
    cache_k[:, :, 9:] = 0
    cache_v[:, :, 9:] = 0
    full = kv_int8_bulk_quantize(cache_k, cache_v, None)
    part = kv_int8_bulk_quantize(cache_k, cache_v, 5)
    out.update(kv_row=_np(row), kv_row_codes=_np(c), kv_row_scale=_np(s),
               kv_cache_k=_np(cache_k), kv_cache_v=_np(cache_v))
    for tag, d in (("full", full), ("part", part)):
        for name in ("kc", "ks", "vc", "vs"):
            out["kv_bulk_%s_%s" % (tag, name)] = _np(d[name])


def gen_attention(out):
    from lemoq.kernels.attn_decode import dense_attention_oracle, split_kv_oracle
    from lemoq.kernels.kv_int8 import dequant_int8, quantize_per_token_int8

    g = torch.Generator().manual_seed(15)
    q = torch.randn(1, 4, 1, 64, generator=g).half()
    k = torch.randn(1, 4, 40, 64, generator=g).half()
    v = torch.randn(1, 4, 40, 64, generator=g).half()
    out.update(attn_q=_np(q), attn_k=_np(k), attn_v=_np(v))
    for n in (0, 1, 17, 40):
        out["attn_dense_%d" % n] = _np(dense_attention_oracle(q, k, v, n))
        out["attn_split3_%d" % n] = _np(split_kv_oracle(q, k, v, n, num_splits=3, block_n=8))
    kc, ks = quantize_per_token_int8(k)
    vc, vs = quantize_per_token_int8(v)
    kd = dequant_int8(kc, ks.unsqueeze(-1))
    vd = dequant_int8(vc, vs.unsqueeze(-1))
    out.update(attn_kc=_np(kc), attn_ks=_np(ks), attn_vc=_np(vc), attn_vs=_np(vs))
    for n in (1, 17, 40):
        out["attn_int8_%d" % n] = _np(dense_attention_oracle(q, kd, vd, n))


def gen_routing(out):
    from lemoq.kernels.moe_static import _route

    os.environ["LEMOQ_FUSED_ROUTE"] = "0"
    g = torch.Generator().manual_seed(16)
    x = torch.randn(3, 256, generator=g)
    rw = torch.randn(16, 256, generator=g) * 0.05
    logits, top_w, top_i = _route(x, rw, top_k=4, norm_topk_prob=False)
    _, top_wn, top_in = _route(x, rw, top_k=4, norm_topk_prob=True)
    out.update(route_x=_np(x), route_w=_np(rw), route_logits=_np(logits), route_top_w=_np(top_w),
               route_top_i=_np(top_i), route_top_w_norm=_np(top_wn), route_top_i_norm=_np(top_in))
    # 64 experts / top 8 on fp16-valued logits (what the decode step feeds the kernel)
    lg = torch.randn(5, 64, generator=g).half().float()
    w64 = torch.softmax(lg, dim=-1, dtype=torch.float)
    tw, ti = torch.topk(w64, 8, dim=-1)
    out.update(route64_logits=_np(lg), route64_top_w=_np(tw), route64_top_i=_np(ti))
    del os.environ["LEMOQ_FUSED_ROUTE"]


def gen_hf_pieces(out):
    """RMSNorm, rotary tables and apply_rotary of the transformers OLMoE implementation."""
    from transformers import OlmoeConfig
    from transformers.models.olmoe.modeling_olmoe import (
        OlmoeRMSNorm,
        OlmoeRotaryEmbedding,
        apply_rotary_pos_emb,
    )

    g = torch.Generator().manual_seed(17)
    x = (torch.randn(3, 256, generator=g) * 1.7).half()
    w = (torch.randn(256, generator=g) * 0.5 + 1.0).half()
    norm = OlmoeRMSNorm(256, eps=1e-5)
    norm.weight.data = w.clone()
    out.update(norm_x=_np(x), norm_w=_np(w), norm_y=_np(norm(x)))

    cfg = OlmoeConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=4, rope_theta=10000.0,
                      max_position_embeddings=4096)
    rot = OlmoeRotaryEmbedding(cfg)
    pos = torch.tensor([[0, 1, 7, 1024, 1055, 4095, 4127]])
    cos, sin = rot(torch.zeros(1, dtype=torch.float16), pos)
    out.update(rope_positions=_np(pos[0]), rope_cos=_np(cos[0]), rope_sin=_np(sin[0]))

    q = torch.randn(1, 4, 1, 64, generator=g)
    k = torch.randn(1, 4, 1, 64, generator=g)
    c32, s32 = rot(torch.zeros(1, dtype=torch.float32), torch.tensor([[1033]]))
    qo, ko = apply_rotary_pos_emb(q, k, c32, s32)
    out.update(rope_q=_np(q), rope_k=_np(k), rope_c=_np(c32), rope_s=_np(s32), rope_qo=_np(qo), rope_ko=_np(ko))


def gen_hf_model(out):
    """A tiny fp32 OlmoeForCausalLM: weights, a prompt, and greedy logits computed by
    re-running the full forward on the growing prefix (no cache involved)."""
    from transformers import OlmoeConfig, OlmoeForCausalLM

    torch.manual_seed(18)
    cfg = OlmoeConfig(vocab_size=96, hidden_size=64, intermediate_size=32, num_hidden_layers=2,
                      num_attention_heads=2, num_key_value_heads=2, num_experts=4, num_experts_per_tok=2,
                      rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=64,
                      norm_topk_prob=False, tie_word_embeddings=False, attn_implementation="eager")
    model = OlmoeForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 1:  # norm weights: make them matter
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
            else:
                p.copy_(torch.randn_like(p) * 0.05)
    sd = model.state_dict()
    for name, t in sd.items():
        out["hf_w/" + name] = _np(t)
    ids = torch.tensor([[5, 17, 3, 90, 41, 7]])
    logits = []
    tokens = []
    with torch.no_grad():
        cur = ids
        for _ in range(5):
            lg = model(cur, use_cache=False).logits[0, -1]
            logits.append(lg)
            nxt = int(lg.argmax())
            tokens.append(nxt)
            cur = torch.cat([cur, torch.tensor([[nxt]])], dim=1)
    out.update(hf_prompt=_np(ids[0]), hf_logits=_np(torch.stack(logits)), hf_tokens=np.array(tokens))


def gen_layer_trace(out):
    """One W8 decoder-layer decode step assembled from the reference's op functions
    (the reference's own model wrapper needs transformers 4.57 and cannot run here):
    dense projections through dequant_gemm_separate_reference, KV quantisation through
    quantize_per_token_int8, attention through dense_attention_oracle on the dequantised
    mirror, the MoE block through static_moe_forward_grouped_quant(backend="oracle")."""
    from lemoq.kernels.attn_decode import dense_attention_oracle
    from lemoq.kernels.kv_int8 import dequant_int8, kv_int8_bulk_quantize, quantize_per_token_int8
    from lemoq.kernels.moe_grouped_quant import quantize_fused_experts, static_moe_forward_grouped_quant
    from lemoq.kernels.moe_static import FusedExperts
    from lemoq.kernels.reference import dequant_gemm_separate_reference
    from lemoq.quant import rtn
    from transformers import OlmoeConfig
    from transformers.models.olmoe.modeling_olmoe import OlmoeRMSNorm, OlmoeRotaryEmbedding, apply_rotary_pos_emb

    g = torch.Generator().manual_seed(19)
    hidden, heads, hd, e, f, k = 128, 2, 64, 4, 128, 2
    pos, cap = 9, 16

    def q8(w):
        q = rtn.quantize_rtn(w.float(), bits=8, group_size=128, symmetric=True)
        return q["codes"].to(torch.int8), q["scale"].half()

    def lin(x, cs):
        return dequant_gemm_separate_reference(x, cs[0], cs[1], None, group_size=128, out_dtype=torch.float16)

    def norm(x, w):
        m = OlmoeRMSNorm(x.shape[-1], eps=1e-5)
        m.weight.data = w.clone()
        return m(x)

    wq, wk, wv, wo = (torch.randn(hidden, hidden, generator=g) * 0.05 for _ in range(4))
    ln1, ln2, qn, kn = ((1 + 0.1 * torch.randn(hidden, generator=g)).half() for _ in range(4))
    router = (torch.randn(e, hidden, generator=g) * 0.05).half()
    gate_up = (torch.randn(e, 2 * f, hidden, generator=g) * 0.05).half()
    down = (torch.randn(e, hidden, f, generator=g) * 0.05).half()
    qkv = q8(torch.cat((wq, wk, wv), dim=0))
    o8 = q8(wo)
    qexp = quantize_fused_experts(FusedExperts(gate_up=gate_up, down=down), bits=8, group_size=128)
    x = torch.randn(1, hidden, generator=g).half()
    keys = torch.zeros(1, heads, cap, hd).half()
    values = torch.zeros(1, heads, cap, hd).half()
    keys[:, :, :pos] = torch.randn(1, heads, pos, hd, generator=g).half()
    values[:, :, :pos] = torch.randn(1, heads, pos, hd, generator=g).half()
    out.update({"lt/" + n: _np(t) for n, t in dict(
        qkv_codes=qkv[0], qkv_scale=qkv[1], o_codes=o8[0], o_scale=o8[1], ln1=ln1, ln2=ln2, q_norm=qn,
        k_norm=kn, router=router, gu_codes=qexp.packed_gate_up, gu_scale=qexp.scale_gate_up,
        dn_codes=qexp.packed_down, dn_scale=qexp.scale_down, x=x, keys=keys, values=values).items()})

    h = norm(x, ln1)
    y = lin(h, qkv)
    qs, ks_, vs_ = y[:, :hidden], y[:, hidden:2 * hidden], y[:, 2 * hidden:]
    qs, ks_ = norm(qs, qn), norm(ks_, kn)
    qh = qs.view(1, 1, heads, hd).transpose(1, 2)
    kh = ks_.view(1, 1, heads, hd).transpose(1, 2)
    vh = vs_.view(1, 1, heads, hd).transpose(1, 2)
    cfg = OlmoeConfig(hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=heads,
                      rope_theta=10000.0, max_position_embeddings=4096)
    cos, sin = OlmoeRotaryEmbedding(cfg)(torch.zeros(1, dtype=torch.float16), torch.tensor([[pos]]))
    # fused-RoPE semantics (src/lemoq/kernels/rope.py:101-123): fp32 math, one rounding
    qr, kr = apply_rotary_pos_emb(qh.float(), kh.float(), cos.float(), sin.float())
    qr, kr = qr.half(), kr.half()
    bufs = kv_int8_bulk_quantize(keys, values, None)
    keys[:, :, pos:pos + 1] = kr
    values[:, :, pos:pos + 1] = vh
    kc, ksc = quantize_per_token_int8(kr)
    vc, vsc = quantize_per_token_int8(vh)
    bufs["kc"][:, :, pos:pos + 1], bufs["ks"][:, :, pos:pos + 1] = kc, ksc
    bufs["vc"][:, :, pos:pos + 1], bufs["vs"][:, :, pos:pos + 1] = vc, vsc
    kd = dequant_int8(bufs["kc"], bufs["ks"].unsqueeze(-1))
    vd = dequant_int8(bufs["vc"], bufs["vs"].unsqueeze(-1))
    attn = dense_attention_oracle(qr, kd, vd, pos + 1).half().reshape(1, hidden)
    o = lin(attn, o8)
    x1 = x + o
    h2 = norm(x1, ln2)
    moe, logits = static_moe_forward_grouped_quant(h2.reshape(1, 1, hidden), router, qexp, top_k=k,
                                                   norm_topk_prob=False, act_fn=None, backend="oracle")
    x2 = x1 + moe.reshape(1, hidden)
    out.update({"lt/" + n: _np(t) for n, t in dict(
        pos=torch.tensor(pos), h=h, qkv=y, q_rope=qr, k_rope=kr, kc=bufs["kc"], ks=bufs["ks"], vc=bufs["vc"],
        vs=bufs["vs"], keys_after=keys, values_after=values, attn=attn, o=o, x1=x1, h2=h2,
        router_logits=logits.reshape(-1), moe=moe.reshape(-1), x2=x2).items()})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its src/ is put on sys.path)")
    args = ap.parse_args()
    sys.path[:0] = [os.path.join(args.reference, "src"), args.reference]
    torch.set_num_threads(1)  # fixed reduction order inside the generators
    ops, model = {}, {}
    for fn in (gen_rtn, gen_experts, gen_dense, gen_kv, gen_attention, gen_routing, gen_hf_pieces,
               gen_layer_trace):
        fn(ops)
    gen_hf_model(model)
    np.savez_compressed(os.path.join(HERE, "ops_golden.npz"), **ops)
    np.savez_compressed(os.path.join(HERE, "hf_tiny_model_golden.npz"), **model)
    for name in ("ops_golden.npz", "hf_tiny_model_golden.npz"):
        print(name, os.path.getsize(os.path.join(HERE, name)), "bytes")


if __name__ == "__main__":
    main()
