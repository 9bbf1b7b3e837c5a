"""Helpers shared by the GPU parity tests (imports the oracle: test infrastructure only)."""

from __future__ import annotations

import numpy as np
import torch

from oracle import lemoq_oracle as ops
from oracle import olmoe_decode_oracle as glue


def T(a, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def rel_err(got, ref):
    """max |got - ref| / max |ref| -- the 'relative error' of the per-kernel gate (2e-3)."""
    got, ref = got.detach().double().cpu().reshape(-1), ref.detach().double().cpu().reshape(-1)
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-12))


PER_KERNEL_REL_TOL = 2e-3  # the stated parity gates: per-kernel fp16 outputs within 2e-3 relative error


def lemoq_model_from_oracle(w: glue.ModelWeights, device="cuda"):
    """Build the product's module tree (fp16, on the GPU) from unquantised oracle weights."""
    from lemoq.model import OlmoeConfig, OlmoeForCausalLM

    sp = w.spec
    cfg = OlmoeConfig(vocab_size=sp.vocab, hidden_size=sp.hidden, intermediate_size=sp.ffn, num_hidden_layers=sp.layers,
                      num_attention_heads=sp.heads, num_key_value_heads=sp.heads, num_experts=sp.experts,
                      num_experts_per_tok=sp.top_k, rms_norm_eps=sp.eps, rope_theta=sp.rope_theta,
                      norm_topk_prob=sp.norm_topk_prob)
    with torch.device(device):
        model = OlmoeForCausalLM(cfg).to(torch.float16).eval()
    a, f = sp.attn_dim, sp.ffn
    with torch.no_grad():
        model.model.embed_tokens.weight.copy_(w.embed)
        model.model.norm.weight.copy_(w.final_norm)
        model.lm_head.weight.copy_(w.lm_head_w)
        for layer, lw in zip(model.model.layers, w.layers):
            layer.input_layernorm.weight.copy_(lw.ln1)
            layer.post_attention_layernorm.weight.copy_(lw.ln2)
            at = layer.self_attn
            at.q_proj.weight.copy_(lw.qkv_w[:a])
            at.k_proj.weight.copy_(lw.qkv_w[a:2 * a])
            at.v_proj.weight.copy_(lw.qkv_w[2 * a:])
            at.o_proj.weight.copy_(lw.o_w)
            at.q_norm.weight.copy_(lw.q_norm)
            at.k_norm.weight.copy_(lw.k_norm)
            layer.mlp.gate.weight.copy_(lw.router)
            for e, ex in enumerate(layer.mlp.experts):
                ex.gate_proj.weight.copy_(lw.gate_up_w[e, :f])
                ex.up_proj.weight.copy_(lw.gate_up_w[e, f:])
                ex.down_proj.weight.copy_(lw.down_w[e])
    return model


def install_canonical(model, ctx, max_new_tokens):
    """The canonical cell's install order (W8A16 g128 + lm_head W8, kernel attention, grouped MoE)."""
    from benchmarks.runner import install_replacements

    return install_replacements(model, attn="kernel", moe="grouped",
                                quant_cfg={"bit_width": "w8a16", "dequant": "fused", "group_size": 128},
                                rmsnorm="fused", ctx=ctx, max_new_tokens=max_new_tokens)


def oracle_weights_from_model(model, spec: glue.OlmoeSpec) -> glue.ModelWeights:
    """Pull the product's quantised tensors back to the CPU as oracle weights (codes are the product's:
    their bit-exactness against the oracle quantiser is tested separately)."""
    layers = []
    for layer in model.model.layers:
        at, mlp = layer.self_attn, layer.mlp
        ex = mlp._static_experts
        pk = at._lemoq_packed_qkv
        layers.append(glue.LayerWeights(
            ln1=layer.input_layernorm.weight.detach().cpu(), ln2=layer.post_attention_layernorm.weight.detach().cpu(),
            q_norm=at.q_norm.weight.detach().cpu(), k_norm=at.k_norm.weight.detach().cpu(),
            router=mlp._static_router.detach().cpu(),
            qkv_codes=pk.packed.cpu(), qkv_scale=pk.scale.cpu(), o_codes=at.o_proj.packed.cpu(), o_scale=at.o_proj.scale.cpu(),
            experts=ops.QuantExperts(ex.packed_gate_up.cpu(), ex.scale_gate_up.cpu(), ex.packed_down.cpu(),
                                     ex.scale_down.cpu(), ex.group_size)))
    return glue.ModelWeights(spec=spec, embed=model.model.embed_tokens.weight.detach().cpu(), layers=layers,
                             final_norm=model.model.norm.weight.detach().cpu(),
                             lm_head_codes=model.lm_head.packed.cpu(), lm_head_scale=model.lm_head.scale.cpu(), quantized=True)


def oracle_state_from_session(session, spec: glue.OlmoeSpec) -> glue.DecodeState:
    """Copy the session's fp16 caches to an oracle state and build its int8 mirror with the oracle."""
    st = glue.new_state(spec, session.config.max_cache_len)
    for i, cl in enumerate(session.cache.layers):
        st.keys[i].copy_(cl.keys.cpu())
        st.values[i].copy_(cl.values.cpu())
    glue.build_int8_mirror(st)
    return st
