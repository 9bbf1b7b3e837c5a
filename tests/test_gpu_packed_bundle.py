"""A model whose experts come from a packed bundle decodes exactly like the model quantised at start-up: the same
codes (bit for bit), hence the same logits and tokens through the whole-step engine."""

from __future__ import annotations

import pytest
import torch

from gpu_util import install_canonical, lemoq_model_from_oracle
from oracle import olmoe_decode_oracle as glue

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_bundle_loaded_model_equals_the_model_quantised_at_start_up(tmp_path):
    from benchmarks.cudagraph import StaticCacheDecodeSession
    from benchmarks.runner import install_replacements
    from lemoq.quant.expert_calibration import export_rtn_bundle, load_bundle

    spec = glue.OlmoeSpec(layers=2, hidden=512, heads=4, head_dim=128, experts=8, top_k=2, ffn=512, vocab=1024)
    ctx, new = 48, 8
    wf = glue.random_float_weights(spec, seed=21, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    prompt = torch.tensor([[(5 * i + 2) % spec.vocab for i in range(ctx)]], device=DEV)

    direct = lemoq_model_from_oracle(wf)
    install_canonical(direct, ctx, new)

    donor = lemoq_model_from_oracle(wf)
    manifest = export_rtn_bundle(donor, tmp_path, model_id="small-olmoe", group_size=128)
    assert manifest["status"] == "complete" and len(manifest["layers"]) == spec.layers
    assert all(hasattr(layer.mlp, "experts") for layer in donor.model.layers)  # exporting does not modify the model
    loaded_model = lemoq_model_from_oracle(wf)
    bundle = load_bundle(tmp_path, loaded_model, expected_model_id="small-olmoe")
    info = install_replacements(loaded_model, attn="kernel", moe="grouped",
                                quant_cfg={"bit_width": "w8a16", "dequant": "fused", "group_size": 128}, rmsnorm="fused",
                                ctx=ctx, max_new_tokens=new, prequantized=bundle)
    assert info["experts_from_bundle"] and info["moe_replaced"] == spec.layers
    for a, b in zip(direct.model.layers, loaded_model.model.layers):
        for name in ("packed_gate_up", "scale_gate_up", "packed_down", "scale_down"):
            got = getattr(b.mlp._static_experts, name)
            assert got.is_cuda and torch.equal(getattr(a.mlp._static_experts, name), got), name

    def decode(model):
        session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=new, engine="step")
        session.capture(warmup=1)
        assert session.capture_info["step_kernel"] == "whole-step"
        session.reset()
        tokens, logits = [], []
        for _ in range(new):
            session.replay(synchronize=True)
            tokens.append(session.current_token_id)
            logits.append(session.logits_cpu())
        session.close()
        return tokens, logits

    want_tokens, want_logits = decode(direct)
    got_tokens, got_logits = decode(loaded_model)
    assert got_tokens == want_tokens
    assert all(torch.equal(a, b) for a, b in zip(want_logits, got_logits))
