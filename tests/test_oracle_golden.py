"""Pin the CPU oracle against vectors produced by the reference itself
(tests/golden/make_golden.py).  Integer results must match bit for bit."""

from __future__ import annotations

import numpy as np
import torch

from oracle import lemoq_oracle as ops
from oracle import olmoe_decode_oracle as glue


def T(a):
    return torch.from_numpy(np.asarray(a))


def test_rtn_codes_and_scales_bit_exact(ops_golden):
    g = ops_golden
    codes, scale = ops.rtn_quantize_w8(T(g["rtn_w"]), 128)
    assert torch.equal(codes, T(g["rtn_codes"]))
    assert torch.equal(scale, T(g["rtn_scale_fp16"]))
    # half-to-even and the zero group really are in the fixture
    assert (T(g["rtn_scale_fp32"])[3, 1] == 1.0) and int(T(g["rtn_codes"])[3, 128:].abs().max()) == 0
    assert T(g["rtn_codes"])[7, 1:9].tolist() == [0, 2, 2, 4, 0, -2, -2, 126]


def test_expert_quantisation_bit_exact(ops_golden):
    g = ops_golden
    q = ops.quantize_experts(T(g["moe_gate_up"]), T(g["moe_down"]), 128)
    assert torch.equal(q.packed_gate_up, T(g["moe_gu_codes"]))
    assert torch.equal(q.scale_gate_up, T(g["moe_gu_scale"]))
    assert torch.equal(q.packed_down, T(g["moe_dn_codes"]))
    assert torch.equal(q.scale_down, T(g["moe_dn_scale"]))


def test_dense_gemv_matches_both_reference_arms(ops_golden):
    g = ops_golden
    y = ops.dense_w8_gemv(T(g["dense_x"]), T(g["dense_codes"]), T(g["dense_scale"]), 128, out_dtype=None)
    assert torch.allclose(y, T(g["dense_y_separate"]), atol=1e-6, rtol=1e-6)
    assert torch.allclose(y, T(g["dense_y_fused"]), atol=1e-5, rtol=1e-5)


def test_kv_quantisation_bit_exact(ops_golden):
    g = ops_golden
    c, s = ops.kv_quantize_per_token(T(g["kv_row"]))
    assert torch.equal(c, T(g["kv_row_codes"]))
    assert torch.equal(s, T(g["kv_row_scale"]))
    assert float(s[0, 2, 0]) == 1.0 and int(c[0, 2].abs().max()) == 0
    # filled=0 takes the reference's whole-cache branch (its test is "filled is not None and filled > 0")
    for tag, filled in (("full", None), ("part", 5), ("full", 0)):
        d = ops.kv_bulk_quantize(T(g["kv_cache_k"]), T(g["kv_cache_v"]), filled)
        for name in ("kc", "ks", "vc", "vs"):
            assert torch.equal(d[name], T(g["kv_bulk_%s_%s" % (tag, name)])), (tag, name)


def test_attention_dense_split_and_int8(ops_golden):
    g = ops_golden
    q, k, v = T(g["attn_q"])[0, :, 0], T(g["attn_k"])[0], T(g["attn_v"])[0]
    for n in (0, 1, 17, 40):
        ref = T(g["attn_dense_%d" % n])
        assert torch.allclose(ops.attention_dense(q, k, v, n), ref, atol=1e-12, rtol=1e-12)
        sp = ops.attention_split_kv(q, k, v, n, num_splits=3, block_n=8)
        assert torch.allclose(sp, T(g["attn_split3_%d" % n]), atol=1e-6, rtol=1e-6)
        assert torch.allclose(sp.double(), ref, atol=1e-5, rtol=1e-5)
    kc, ks, vc, vs = T(g["attn_kc"])[0], T(g["attn_ks"])[0], T(g["attn_vc"])[0], T(g["attn_vs"])[0]
    c2, s2 = ops.kv_quantize_per_token(k)
    assert torch.equal(c2, kc) and torch.equal(s2, ks)
    for n in (1, 17, 40):
        got = ops.attention_int8(q, kc, ks, vc, vs, n)
        # the reference dequantises in fp32 before its fp64 attention
        assert torch.allclose(got, T(g["attn_int8_%d" % n]), atol=1e-6, rtol=1e-6)


def test_routing_ids_bit_exact(ops_golden):
    g = ops_golden
    logits, top_w, top_i = ops.route(T(g["route_x"]), T(g["route_w"]), 4, False)
    assert torch.allclose(logits, T(g["route_logits"]), atol=1e-5, rtol=1e-5)
    assert torch.equal(top_i, T(g["route_top_i"]))
    assert torch.allclose(top_w, T(g["route_top_w"]), atol=1e-6)
    _, top_wn, top_in = ops.route(T(g["route_x"]), T(g["route_w"]), 4, True)
    assert torch.equal(top_in, T(g["route_top_i_norm"]))
    assert torch.allclose(top_wn, T(g["route_top_w_norm"]), atol=1e-6)
    tw, ti = ops.routing_softmax_topk(T(g["route64_logits"]), 8)
    assert torch.equal(ti, T(g["route64_top_i"]))
    assert torch.allclose(tw, T(g["route64_top_w"]), atol=1e-7)


def test_routing_ties_take_lowest_index():
    tw, ti = ops.routing_softmax_topk(torch.zeros(1, 64), 8)
    assert ti.tolist() == [list(range(8))]
    lg = torch.zeros(1, 64)
    lg[0, :7] = torch.arange(8, 1, -1).float()
    _, ti = ops.routing_softmax_topk(lg, 8)
    assert ti.tolist() == [[0, 1, 2, 3, 4, 5, 6, 7]]


def test_grouped_moe_matches_reference_oracle_backend(ops_golden):
    g = ops_golden
    q = ops.QuantExperts(T(g["moe_gu_codes"]), T(g["moe_gu_scale"]), T(g["moe_dn_codes"]), T(g["moe_dn_scale"]), 128)
    out, _ = ops.grouped_moe_w8(T(g["moe_x"]), q, T(g["moe_ids"]), T(g["moe_top_w"]))
    ref = T(g["moe_out_w8"])
    assert out.dtype == torch.float16
    assert torch.allclose(out.float(), ref.float(), atol=2e-3 * float(ref.float().abs().max()), rtol=0)
    # fp16 ulp-level agreement: same maths, only the matmul blocking differs
    assert float((out.float() - ref.float()).abs().max()) <= 2.0 ** -10 * float(ref.float().abs().max())
    out16, _ = ops.grouped_moe_fp16(T(g["moe_x"]), T(g["moe_gate_up"]), T(g["moe_down"]), T(g["moe_ids"]),
                                    T(g["moe_top_w"]))
    ref16 = T(g["moe_out_fp16"])
    assert float((out16.float() - ref16.float()).abs().max()) <= 2.0 ** -10 * float(ref16.float().abs().max())
    blk, logits, top_w, top_i = ops.moe_block_w8(T(g["moe_x"]), T(g["moe_router"]), q, 2)
    assert torch.allclose(logits.float(), T(g["moe_block_logits"]).float(), atol=1e-3)
    refb = T(g["moe_block_out"]).float()
    assert float((blk.float() - refb).abs().max()) <= 2.0 ** -10 * float(refb.abs().max())


def test_rmsnorm_and_rope_match_transformers(ops_golden):
    g = ops_golden
    y = ops.rms_norm(T(g["norm_x"]), T(g["norm_w"]), 1e-5)
    assert torch.equal(y, T(g["norm_y"]))
    cos, sin = ops.rope_tables(4128, 64)
    pos = T(g["rope_positions"]).long()
    assert torch.equal(cos[pos], T(g["rope_cos"]))
    assert torch.equal(sin[pos], T(g["rope_sin"]))
    qo = ops.apply_rope(T(g["rope_q"])[0, :, 0], T(g["rope_c"])[0], T(g["rope_s"])[0])
    ko = ops.apply_rope(T(g["rope_k"])[0, :, 0], T(g["rope_c"])[0], T(g["rope_s"])[0])
    assert torch.allclose(qo, T(g["rope_qo"])[0, :, 0], atol=1e-6)
    assert torch.allclose(ko, T(g["rope_ko"])[0, :, 0], atol=1e-6)


def _layer_from_fixture(g):
    spec = glue.OlmoeSpec(layers=1, hidden=128, heads=2, head_dim=64, experts=4, top_k=2, ffn=128, vocab=8)
    ex = ops.QuantExperts(T(g["lt/gu_codes"]), T(g["lt/gu_scale"]), T(g["lt/dn_codes"]), T(g["lt/dn_scale"]), 128)
    lw = glue.LayerWeights(ln1=T(g["lt/ln1"]), ln2=T(g["lt/ln2"]), q_norm=T(g["lt/q_norm"]), k_norm=T(g["lt/k_norm"]),
                           router=T(g["lt/router"]), qkv_codes=T(g["lt/qkv_codes"]), qkv_scale=T(g["lt/qkv_scale"]),
                           o_codes=T(g["lt/o_codes"]), o_scale=T(g["lt/o_scale"]), experts=ex)
    return spec, lw


def test_one_layer_decode_matches_reference_assembly(ops_golden):
    """The glue (order of ops and rounding points) against a step assembled from the
    reference's own functions."""
    g = ops_golden
    spec, lw = _layer_from_fixture(g)
    pos = int(g["lt/pos"])
    embed = torch.zeros(8, 128, dtype=torch.float16)
    embed[3] = T(g["lt/x"])[0]
    lm_c, lm_s = ops.rtn_quantize_w8(torch.eye(8, 128), 128)
    w = glue.ModelWeights(spec=spec, embed=embed, layers=[lw], final_norm=torch.ones(128, dtype=torch.float16),
                          lm_head_codes=lm_c, lm_head_scale=lm_s, quantized=True)
    st = glue.new_state(spec, 16)
    st.keys[0].copy_(T(g["lt/keys"]))
    st.values[0].copy_(T(g["lt/values"]))
    glue.build_int8_mirror(st)
    trace = {}
    glue.decode_step(w, st, 3, pos, kv_int8=True, trace=trace)
    t = trace["layers"][0]
    assert torch.equal(t["h"].reshape(-1), T(g["lt/h"]).reshape(-1))
    assert torch.equal(t["qkv"].reshape(-1), T(g["lt/qkv"]).reshape(-1))
    assert torch.equal(t["q"], T(g["lt/q_rope"])[0, :, 0])
    assert torch.equal(t["k"], T(g["lt/k_rope"])[0, :, 0])
    for name in ("kc", "ks", "vc", "vs"):
        assert torch.equal(st.mirror[0][name], T(g["lt/" + name])), name
    assert torch.equal(st.keys[0], T(g["lt/keys_after"]))
    assert torch.equal(st.values[0], T(g["lt/values_after"]))

    def close(a, b, ulps=2):
        b = b.reshape(-1).float()
        return float((a.reshape(-1).float() - b).abs().max()) <= ulps * 2.0 ** -11 * max(float(b.abs().max()), 1e-6)

    assert close(t["attn"], T(g["lt/attn"]))
    assert close(t["o"], T(g["lt/o"]))
    assert close(t["x1"], T(g["lt/x1"]))
    assert close(t["h2"], T(g["lt/h2"]), ulps=4)
    assert close(t["router_logits"], T(g["lt/router_logits"]), ulps=4)
    assert close(t["moe"], T(g["lt/moe"]), ulps=4)
    assert close(t["x2"], T(g["lt/x2"]), ulps=4)


def _weights_from_hf(g):
    spec = glue.OlmoeSpec(layers=2, hidden=64, heads=2, head_dim=32, experts=4, top_k=2, ffn=32, vocab=96)
    sd = {k[len("hf_w/"):]: T(v) for k, v in g.items() if k.startswith("hf_w/")}
    layers = []
    for i in range(spec.layers):
        p = "model.layers.%d." % i
        layers.append(glue.LayerWeights(
            ln1=sd[p + "input_layernorm.weight"], ln2=sd[p + "post_attention_layernorm.weight"],
            q_norm=sd[p + "self_attn.q_norm.weight"], k_norm=sd[p + "self_attn.k_norm.weight"],
            router=sd[p + "mlp.gate.weight"],
            qkv_w=torch.cat([sd[p + "self_attn.%s_proj.weight" % n] for n in "qkv"], dim=0),
            o_w=sd[p + "self_attn.o_proj.weight"],
            gate_up_w=sd[p + "mlp.experts.gate_up_proj"], down_w=sd[p + "mlp.experts.down_proj"]))
    return glue.ModelWeights(spec=spec, embed=sd["model.embed_tokens.weight"], layers=layers,
                             final_norm=sd["model.norm.weight"], lm_head_w=sd["lm_head.weight"], quantized=False)


def test_glue_matches_transformers_olmoe_fp32(hf_golden):
    """Prefill + cached greedy decode of the restated glue against transformers' own
    OlmoeForCausalLM re-run on the growing prefix (fp32, unquantised)."""
    g = hf_golden
    w = _weights_from_hf(g)
    prompt = T(g["hf_prompt"]).long()
    ref_logits = T(g["hf_logits"])
    st = glue.new_state(w.spec, 32, dtype=torch.float32)
    first = glue.prefill(w, st, prompt)
    assert torch.allclose(first, ref_logits[0], atol=2e-5, rtol=1e-4)
    tok = int(first.argmax())
    assert tok == int(g["hf_tokens"][0])
    toks, logits = glue.greedy_decode(w, st, tok, int(prompt.numel()), 4, kv_int8=False)
    for i in range(4):
        assert torch.allclose(logits[i], ref_logits[i + 1], atol=2e-5, rtol=1e-4), i
    assert toks == [int(t) for t in g["hf_tokens"][1:]]


def test_compare_logits_gate():
    a = [torch.randn(1, 50) for _ in range(3)]
    rep = ops.compare_logits(a, a)
    assert rep["kl"] == 0.0 and rep["top1_agreement"] == 1.0
    b = [x + 0.5 * torch.randn_like(x) for x in a]
    assert ops.compare_logits(a, b)["kl"] > 1e-3
