"""CPU-side tests: the C-ABI library loads and exports every declared symbol, host-side
contracts raise the right exception types before any kernel call, switches, byte model, runner
refusals, and the module tree's glue against transformers' OLMoE (golden logits)."""

from __future__ import annotations

import os
import re

import numpy as np
import pytest
import torch

from conftest import PKG, ROOT


def test_library_exports_every_declared_symbol():
    from lemoq import _cabi

    header = open(os.path.join(ROOT, "include", "lemoq_b200.h")).read()
    declared = set(re.findall(r"LEMOQ_API[^;(]*?\b(lemoq_\w+)\s*\(", header))
    assert len(declared) >= 20
    assert declared == set(_cabi.EXPORTED_SYMBOLS), declared ^ set(_cabi.EXPORTED_SYMBOLS)
    lib = _cabi.lib()  # fails loudly if the .so is missing
    for name in declared:
        assert hasattr(lib, name), name
    assert b"sm_100a" in lib.lemoq_version()


def test_header_cites_a_reference_interface_for_every_entry_point():
    header = open(os.path.join(ROOT, "include", "lemoq_b200.h")).read()
    blocks = header.split("/* -----")
    for block in blocks[1:]:
        if "LEMOQ_API" in block:
            # every entry point cites the reference interface it replaces, or says that it has none
            assert "ref:" in block or "no counterpart in the\n * reference" in block or "no counterpart in the reference" in block, block[:200]


def test_cabi_argument_validation_needs_no_gpu():
    from lemoq import _cabi

    lib = _cabi.lib()
    # null pointers / bad sizes are rejected before any CUDA call
    assert lib.lemoq_rms_norm(None, None, None, 1, 2048, 1e-5, None) == _cabi.ERR_INVALID
    assert "null" in _cabi.last_error()
    assert lib.lemoq_rtn_quantize_w8(1 << 20, 0, 4, 100, 128, 1 << 21, 1 << 22, None) == _cabi.ERR_UNSUPPORTED
    assert lib.lemoq_attn_decode_int8(16, 16, 16, 16, 16, 128, 16, 16, 2, 8, 48, 2, 0.1, 16, None, None) == _cabi.ERR_UNSUPPORTED
    assert "head_dim" in _cabi.last_error()
    assert lib.lemoq_routing_softmax_topk(16, 0, 64, 1, 64, 65, 0, 16, 16, None) == _cabi.ERR_INVALID
    assert lib.lemoq_attn_workspace_bytes(16, 128, 10) == 256 + 4 * 16 * 10 * 130
    with pytest.raises(ValueError):
        _cabi.check(_cabi.ERR_INVALID)
    with pytest.raises(NotImplementedError):
        _cabi.check(_cabi.ERR_UNSUPPORTED)
    with pytest.raises(RuntimeError):
        _cabi.check(_cabi.ERR_CUDA)


def test_ops_refuse_cpu_tensors_instead_of_falling_back():
    from lemoq.kernels.dequant_gemv import dequant_gemm_fused
    from lemoq.kernels.kv_int8 import kv_int8_rows_applicable, quantize_per_token_int8
    from lemoq.kernels.rmsnorm import rms_norm_fused
    from lemoq.kernels.routing import routing_softmax_topk

    if torch.cuda.is_available():
        pytest.skip("error path of a machine without CUDA")
    with pytest.raises(RuntimeError, match="CUDA"):
        routing_softmax_topk(torch.zeros(1, 64), top_k=8)
    with pytest.raises(RuntimeError, match="CUDA"):
        rms_norm_fused(torch.zeros(1, 128, dtype=torch.float16), torch.ones(128, dtype=torch.float16), 1e-5)
    with pytest.raises(RuntimeError, match="CUDA"):
        quantize_per_token_int8(torch.zeros(1, 2, 1, 64, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="CUDA"):
        dequant_gemm_fused(torch.zeros(1, 128, dtype=torch.float16), torch.zeros(4, 128, dtype=torch.int8),
                           torch.ones(4, 1, dtype=torch.float16), group_size=128)
    k = torch.zeros(1, 2, 1, 64, dtype=torch.float16)
    assert kv_int8_rows_applicable(k, k) is False


def test_contract_errors_match_the_reference_types_and_keywords():
    from lemoq.kernels.attn_decode import attn_decode_forward, launch_plan, resolve_num_splits
    from lemoq.kernels.dequant_gemv import dequant_gemm_fused
    from lemoq.kernels.moe_grouped import grouped_moe_forward
    from lemoq.kernels.moe_grouped_quant import QuantFusedExperts, grouped_moe_forward_quant, quant_launch_plan
    from lemoq.kernels.moe_static import FusedExperts, static_moe_forward
    from lemoq.kernels.rmsnorm import rms_norm_fused
    from lemoq.kernels.routing import routing_softmax_topk

    h16 = torch.float16
    with pytest.raises(ValueError, match="weight"):
        rms_norm_fused(torch.zeros(1, 2048, dtype=h16), torch.ones(1024, dtype=h16), 1e-5)
    with pytest.raises(NotImplementedError, match="2 的幂"):
        rms_norm_fused(torch.zeros(1, 1000, dtype=h16), torch.ones(1000, dtype=h16), 1e-5)
    with pytest.raises(ValueError, match="连续"):
        rms_norm_fused(torch.zeros(4, 256, dtype=h16).t().contiguous().t(), torch.ones(4, dtype=h16), 1e-5)
    with pytest.raises(ValueError):
        routing_softmax_topk(torch.zeros(64), top_k=8)
    with pytest.raises(ValueError):
        routing_softmax_topk(torch.zeros(1, 64), top_k=65)
    with pytest.raises(ValueError):
        dequant_gemm_fused(torch.zeros(128, dtype=h16), torch.zeros(4, 128, dtype=torch.int8), torch.ones(4, 1, dtype=h16), group_size=128)
    with pytest.raises(NotImplementedError):
        dequant_gemm_fused(torch.zeros(1, 128, dtype=h16), torch.zeros(4, 64, dtype=torch.uint8), torch.ones(4, 1, dtype=h16),
                           group_size=128, bits=4)
    q = torch.zeros(1, 2, 1, 64, dtype=h16)
    kv = torch.zeros(1, 2, 8, 64, dtype=h16)
    with pytest.raises(NotImplementedError):
        attn_decode_forward(torch.zeros(1, 4, 1, 64, dtype=h16), kv, kv, 3)  # GQA is refused
    with pytest.raises(NotImplementedError):
        attn_decode_forward(torch.zeros(2, 2, 1, 64, dtype=h16), kv, kv, 3)  # batch 2
    with pytest.raises(ValueError):
        attn_decode_forward(q, kv, kv[:, :, :4], 3)
    with pytest.raises(RuntimeError, match="oracle"):
        attn_decode_forward(q, kv, kv, 3, backend="oracle")
    with pytest.raises(ValueError, match="unknown backend"):
        attn_decode_forward(q, kv, kv, 3, backend="bogus")
    with pytest.raises(ValueError):
        launch_plan(heads=16, head_dim=128, num_splits=0)
    assert launch_plan(heads=16, head_dim=128, num_splits=19)["split"]["grid"] == (19, 16)
    assert resolve_num_splits(7, heads=16) == 7
    fused = FusedExperts(gate_up=torch.zeros(4, 256, 128), down=torch.zeros(4, 128, 128))
    with pytest.raises(NotImplementedError, match="fp16"):
        grouped_moe_forward(torch.zeros(128), fused, torch.zeros(2, dtype=torch.long), torch.ones(2))
    qe = QuantFusedExperts(torch.zeros(4, 256, 128, dtype=torch.int8), torch.ones(4, 256, 1), torch.zeros(4, 128, 128, dtype=torch.int8),
                           torch.ones(4, 128, 1), 8, 128)
    with pytest.raises(NotImplementedError, match="fp16"):
        grouped_moe_forward_quant(torch.zeros(128, dtype=h16), qe, torch.zeros(2, dtype=torch.long), torch.ones(2, dtype=h16))
    plan = quant_launch_plan(qe, top_k=2)
    assert plan["hidden"] == 128 and plan["ffn"] == 128 and plan["kernel_count"] == 2
    assert plan["gate_up_act"]["act_shape"] == (2, 128) and plan["down_sum"]["out_shape"] == (128,)
    with pytest.raises(ValueError, match="unknown impl"):
        static_moe_forward(torch.zeros(1, 128), torch.zeros(4, 128), fused, top_k=2, impl="bogus")
    with pytest.raises(ValueError, match="dtype"):
        qe.to(torch.float32)


def test_fusion_switches():
    from lemoq.kernels.fusion_switches import ENV_VARS, FUSION_DEFAULTS, fusion_enabled, fusion_states

    assert set(ENV_VARS) == {"fused_rope", "fused_route", "skip_mask_fill", "packed_qkv", "kv_direct_write", "lm_head_w8", "kv_int8"}
    assert all(FUSION_DEFAULTS.values())
    assert fusion_enabled("kv_int8", env={}) is True
    assert fusion_enabled("kv_int8", env={"LEMOQ_KV_INT8": "0"}) is False
    assert fusion_enabled("kv_int8", env={"LEMOQ_KV_INT8": "yes"}) is False
    assert fusion_enabled("kv_int8", env={"LEMOQ_KV_INT8": "1"}) is True
    with pytest.raises(KeyError, match="未知融合开关"):
        fusion_enabled("nope")
    assert fusion_states(env={"LEMOQ_FUSED_ROPE": "0"})["fused_rope"] is False


def test_byte_model_matches_the_hand_computed_budgets():
    from benchmarks.bytes import CANONICAL_QUANT, ModelSpec, byte_budget, floor_ms, kv_budget, weight_budget

    s = ModelSpec()
    assert weight_budget(s)["total_bytes"] == 2_357_723_136  # fp16 [W], RESULTS.md:100 of the reference
    w8 = {i["name"]: i["bytes"] for i in weight_budget(s, CANONICAL_QUANT)["items"]}
    assert w8 == {"attention": 272_629_760, "router": 4_194_304, "experts(top-k)": 817_889_280, "lm_head": 104_632_320}
    assert byte_budget(s, 1024, CANONICAL_QUANT, True)["T"] == 1_267_503_104
    assert byte_budget(s, 4096, CANONICAL_QUANT, True)["T"] == 1_471_975_424
    assert kv_budget(s, 4096, kv_int8=False)["total_bytes"] == 536_870_912
    assert abs(floor_ms(1_267_503_104, 6552.0) - 0.19345) < 1e-4


def test_runner_refusals_and_cuda_graph_config():
    from benchmarks.cudagraph import CudaGraphConfig, GraphBuffers, normalize_execution
    from benchmarks.runner import Refusal, check_refusals, quant_spec_for_cfg

    base = dict(ctx=1024, batch=1, execution="cudagraph", attn="kernel", moe="grouped", bit_width="fp16", dequant="none",
                group_size=128, rmsnorm="hf", max_new_tokens=32, timed=20)
    check_refusals(**base)
    for patch, word in (({"ctx": 1}, "ctx"), ({"ctx": 4097}, "ctx"), ({"batch": 2}, "batch"),
                        ({"execution": "eager"}, "cudagraph"), ({"bit_width": "w8a16", "moe": "gather"}, "gather"),
                        ({"bit_width": "w8a8"}, "w8a8"), ({"dequant": "fused"}, "quantised"),
                        ({"bit_width": "w8a16", "group_size": 64}, "group_size"), ({"bit_width": "w8a16", "group_size": 127}, "even")):
        with pytest.raises(Refusal, match=word):
            check_refusals(**{**base, **patch})
    with pytest.raises(ValueError, match="unknown execution"):
        normalize_execution("bogus")
    with pytest.raises(ValueError, match="timed"):
        CudaGraphConfig(ctx=16, max_new_tokens=8).validate_timing(20)
    with pytest.raises(ValueError):
        CudaGraphConfig(ctx=1, max_new_tokens=8)
    assert CudaGraphConfig(ctx=1024, max_new_tokens=32).max_cache_len == 1056
    b = GraphBuffers.allocate("cpu", batch=1, max_cache_len=8)
    b.set_step(token=5, position=3)
    assert int(b.filled_len) == 4 and int(b.cache_position) == 3 and b.filled_len.dtype == torch.int32
    spec = quant_spec_for_cfg({"bit_width": "w8a16", "dequant": "fused", "group_size": 128})
    assert spec.targets == ("attention", "experts", "lm_head") and spec.keep_lm_head_fp16 is False and "router" not in spec.targets
    assert quant_spec_for_cfg({"bit_width": "fp16"}) is None


def _load_hf_weights(model, g):
    sd = {k[len("hf_w/"):]: torch.from_numpy(np.asarray(v)) for k, v in g.items() if k.startswith("hf_w/")}
    cfg = model.config
    with torch.no_grad():
        model.model.embed_tokens.weight.copy_(sd["model.embed_tokens.weight"])
        model.model.norm.weight.copy_(sd["model.norm.weight"])
        model.lm_head.weight.copy_(sd["lm_head.weight"])
        for i, layer in enumerate(model.model.layers):
            p = "model.layers.%d." % i
            layer.input_layernorm.weight.copy_(sd[p + "input_layernorm.weight"])
            layer.post_attention_layernorm.weight.copy_(sd[p + "post_attention_layernorm.weight"])
            for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
                getattr(layer.self_attn, n).weight.copy_(sd[p + "self_attn.%s.weight" % n])
            layer.self_attn.q_norm.weight.copy_(sd[p + "self_attn.q_norm.weight"])
            layer.self_attn.k_norm.weight.copy_(sd[p + "self_attn.k_norm.weight"])
            layer.mlp.gate.weight.copy_(sd[p + "mlp.gate.weight"])
            gu, dn = sd[p + "mlp.experts.gate_up_proj"], sd[p + "mlp.experts.down_proj"]
            f = cfg.intermediate_size
            for e, ex in enumerate(layer.mlp.experts):
                ex.gate_proj.weight.copy_(gu[e, :f])
                ex.up_proj.weight.copy_(gu[e, f:])
                ex.down_proj.weight.copy_(dn[e])


def test_module_tree_matches_transformers_olmoe_and_static_cache_decode(hf_golden):
    """The host-side module tree (eager path) against transformers' OlmoeForCausalLM golden logits,
    both by re-running the growing prefix and by StaticCache prefill + one-token decode; then the
    fixed-shape MoE replacement (gather impl) must not change the numbers."""
    from lemoq.kernels.moe_static import replace_moe_blocks
    from lemoq.model import OlmoeConfig, OlmoeForCausalLM, StaticCache

    g = hf_golden
    cfg = OlmoeConfig(vocab_size=96, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=2, num_experts=4, num_experts_per_tok=2, max_position_embeddings=64)
    model = OlmoeForCausalLM(cfg).float().eval()
    _load_hf_weights(model, g)
    prompt = torch.from_numpy(g["hf_prompt"]).long()[None]
    ref = torch.from_numpy(g["hf_logits"])
    toks = [int(t) for t in g["hf_tokens"]]

    def run_cached():
        cache = StaticCache(cfg, 16)
        n = prompt.shape[1]
        pos = torch.arange(n)
        with torch.no_grad():
            out = model(prompt, past_key_values=cache, use_cache=True, cache_position=pos, position_ids=pos[None])
            logits = [out.logits[0, -1]]
            for i in range(4):
                p = torch.tensor([n + i])
                mask = torch.full((1, 1, 1, 16), torch.finfo(torch.float32).min)
                mask[..., : n + i + 1] = 0
                out = model(torch.tensor([[toks[i]]]), attention_mask=mask, past_key_values=cache, use_cache=True,
                            cache_position=p, position_ids=p[None])
                logits.append(out.logits[0, -1])
        return torch.stack(logits)

    with torch.no_grad():
        full = model(torch.cat([prompt, torch.tensor([toks[:4]])], dim=1)).logits[0]
    assert torch.allclose(full[prompt.shape[1] - 1:], ref, atol=2e-5, rtol=1e-4)
    assert torch.allclose(run_cached(), ref, atol=2e-5, rtol=1e-4)
    os.environ["LEMOQ_FUSED_ROUTE"] = "0"
    try:
        assert replace_moe_blocks(model, impl="gather") == 2
        assert not hasattr(model.model.layers[0].mlp, "experts")
        assert torch.allclose(run_cached(), ref, atol=2e-5, rtol=1e-4)
    finally:
        del os.environ["LEMOQ_FUSED_ROUTE"]


def test_quantize_model_classification_rules():
    from lemoq.quant.linear import SchemeSpec, classify_linear

    assert classify_linear("lm_head") == "lm_head"
    assert classify_linear("model.layers.3.self_attn.q_proj") == "attention"
    assert classify_linear("model.layers.3.mlp.experts.17.gate_proj") == "experts"
    assert classify_linear("model.layers.3.mlp.gate") == "router"
    assert classify_linear("model.embed") is None
    with pytest.raises(ValueError, match="dequant"):
        SchemeSpec(dequant="bogus")
    with pytest.raises(NotImplementedError):
        SchemeSpec.from_flags("w4a16", 128)


def test_reference_arm_times_a_bounded_number_of_cpu_steps(monkeypatch, capsys):
    """`bench.py --impl reference`: whatever --steps says, at most REFERENCE_MAX_STEPS CPU decode steps (3 warm-up
    steps) are run, the line keeps the K it was launched with and says how many steps were timed, and its `config`
    is the one the GPU arm prints for the same context."""
    import argparse
    import json
    import sys

    sys.path.insert(0, str(ROOT))
    import bench

    seen = {}

    def fake_steps(wq, st, tok, ctx, steps, warmup):
        seen.update(steps=steps, warmup=warmup, capacity=int(st.keys[0].shape[2]))
        return [0.5] * steps

    monkeypatch.setattr(bench, "synthetic_oracle_weights", lambda spec: None)
    monkeypatch.setattr(bench, "time_oracle_steps", fake_steps)
    monkeypatch.delenv("RANK", raising=False)
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    assert bench.run_reference(argparse.Namespace(steps=400, warmup=5, ctx=64, gpus=1)) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert seen["steps"] == bench.REFERENCE_MAX_STEPS and seen["warmup"] == 3
    assert seen["capacity"] >= 64 + seen["steps"] + seen["warmup"]
    assert line["impl"] == "reference" and line["steps"] == 400 and line["steps_timed"] == bench.REFERENCE_MAX_STEPS
    assert line["value"] == pytest.approx(2.0) and line["ms_per_step"] == pytest.approx(500.0)
    assert line["e2e"]["value"] == line["value"] and line["cpu_baseline"]["kind"] == "port"
    assert str(bench.REFERENCE_MAX_STEPS) in line["cpu_baseline"]["sample"]
    from benchmarks.bytes import CANONICAL_QUANT, ModelSpec, byte_budget
    from lemoq.model import OlmoeConfig

    first = byte_budget(ModelSpec.from_config(OlmoeConfig()), 64 + 1, CANONICAL_QUANT, kv_int8=True)["T"]
    assert line["config"] == bench.workload_config(64, 16, 1, first)
    # a short run is not stretched
    assert bench.run_reference(argparse.Namespace(steps=2, warmup=1, ctx=64, gpus=1)) == 0
    assert seen["steps"] == 2 and seen["warmup"] == 1
    # ranks other than 0 do no work
    monkeypatch.setenv("RANK", "1")
    seen.clear()
    assert bench.run_reference(argparse.Namespace(steps=2, warmup=1, ctx=64, gpus=2)) == 0 and not seen
