"""Packed expert checkpoints on the CPU: write / load round trip, every refusal of the loader and of
``replace_moe_blocks(prequantized=...)`` (an invalid payload leaves the model untouched), as the reference's
tests/test_expert_calibration.py checks them.  The containers are built with the oracle's quantiser."""

from __future__ import annotations

import json

import pytest
import torch

from oracle import lemoq_oracle as ops

GROUP = 4


def tiny_model():
    from lemoq.model import OlmoeConfig, OlmoeForCausalLM

    torch.manual_seed(3)
    cfg = OlmoeConfig(vocab_size=32, hidden_size=16, intermediate_size=8, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=2, num_experts=2, num_experts_per_tok=1)
    return OlmoeForCausalLM(cfg).eval()


def containers_of(model):
    from lemoq.kernels.moe_grouped_quant import QuantFusedExperts
    from lemoq.kernels.moe_static import fuse_experts

    out = {}
    for i, layer in enumerate(model.model.layers):
        fused = fuse_experts(layer.mlp.experts)
        gc, gs = ops.rtn_quantize_w8(fused.gate_up.reshape(-1, fused.gate_up.shape[-1]).float(), GROUP)
        dc, ds = ops.rtn_quantize_w8(fused.down.reshape(-1, fused.down.shape[-1]).float(), GROUP)
        e = fused.num_experts
        out[i] = QuantFusedExperts(gc.reshape(e, -1, gc.shape[-1]).contiguous(), gs.reshape(e, -1, gs.shape[-1]).contiguous(),
                                   dc.reshape(e, -1, dc.shape[-1]).contiguous(), ds.reshape(e, -1, ds.shape[-1]).contiguous(), 8, GROUP)
    return out


def test_round_trip_and_install(tmp_path):
    from lemoq.kernels.moe_static import replace_moe_blocks
    from lemoq.quant.expert_calibration import file_sha256, load_bundle, validate_packed, write_bundle

    model = tiny_model()
    packed = containers_of(model)
    manifest = write_bundle(tmp_path, packed, model_id="tiny-olmoe")
    assert manifest["status"] == "complete" and [r["layer"] for r in manifest["layers"]] == [0, 1]
    assert all(file_sha256(tmp_path / r["file"]) == r["sha256"] for r in manifest["layers"])
    with pytest.raises(FileExistsError):  # a bundle file is never overwritten
        write_bundle(tmp_path, packed, model_id="tiny-olmoe")
    loaded = load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")
    for i, q in loaded.items():
        validate_packed(q, experts=2, hidden=16, ffn=8)
        for name in ("packed_gate_up", "scale_gate_up", "packed_down", "scale_down"):
            assert torch.equal(getattr(q, name), getattr(packed[i], name))
        assert (q.bits, q.group_size) == (8, GROUP)
    x = torch.randn(1, 3, 16)
    assert replace_moe_blocks(model, impl="grouped", prequantized=loaded) == 2
    for i, layer in enumerate(model.model.layers):
        assert not hasattr(layer.mlp, "experts") and layer.mlp._static_experts.packed_down.data_ptr() == loaded[i].packed_down.data_ptr()
        y, logits = layer.mlp(x)  # several tokens: the eager path dequantises the loaded codes
        assert y.shape == x.shape and logits.shape == (3, 2) and bool(torch.isfinite(y).all())
    # a model whose experts are already fused can still be matched against a bundle
    assert set(load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")) == {0, 1}


def test_invalid_payload_is_refused_before_any_block_is_touched():
    from lemoq.kernels.moe_static import replace_moe_blocks

    model = tiny_model()
    packed = containers_of(model)
    packed[1].scale_down[0, 0, 0] = float("nan")
    with pytest.raises(ValueError, match="scales"):
        replace_moe_blocks(model, impl="grouped", prequantized=packed)
    assert all(hasattr(layer.mlp, "experts") for layer in model.model.layers)
    with pytest.raises(ValueError, match="cover all model layers"):
        replace_moe_blocks(model, impl="grouped", prequantized={0: packed[0]})
    with pytest.raises(ValueError, match="prequantized requires grouped"):
        replace_moe_blocks(model, impl="gather", prequantized=packed)


def test_validate_packed_rules():
    from lemoq.quant.expert_calibration import validate_packed

    q = containers_of(tiny_model())[0]
    validate_packed(q, experts=2, hidden=16, ffn=8)
    q.scale_down[0, 0, 0] = 0  # an fp32 scale that underflowed in fp16 is valid
    validate_packed(q, experts=2, hidden=16, ffn=8)
    q.scale_down[0, 0, 0] = -1
    with pytest.raises(ValueError, match="scales"):
        validate_packed(q, experts=2, hidden=16, ffn=8)
    q.scale_down[0, 0, 0] = 1
    with pytest.raises(ValueError, match="mismatch: packed_gate_up"):
        validate_packed(q, experts=3, hidden=16, ffn=8)
    with pytest.raises(ValueError, match="group size must divide"):
        validate_packed(q, experts=2, hidden=18, ffn=8)
    q.packed_down = q.packed_down.to(torch.int16)
    with pytest.raises(ValueError, match="mismatch: packed_down"):
        validate_packed(q, experts=2, hidden=16, ffn=8)
    q.bits = 3
    with pytest.raises(ValueError, match="container"):
        validate_packed(q, experts=2, hidden=16, ffn=8)
    with pytest.raises(ValueError, match="container"):
        validate_packed(object(), experts=2, hidden=16, ffn=8)


def test_loader_refusals(tmp_path):
    from lemoq.quant.expert_calibration import MANIFEST, load_bundle, write_bundle

    model = tiny_model()
    write_bundle(tmp_path, containers_of(model), model_id="tiny-olmoe")
    text = (tmp_path / MANIFEST).read_text()

    def with_manifest(change):
        m = json.loads(text)
        change(m)
        (tmp_path / MANIFEST).write_text(json.dumps(m))

    with pytest.raises(ValueError, match="identity"):
        load_bundle(tmp_path, model, expected_model_id="another-model")
    with_manifest(lambda m: m.update(status="partial"))
    with pytest.raises(ValueError, match="incomplete"):
        load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")
    with_manifest(lambda m: m["layers"].pop())
    with pytest.raises(ValueError, match="every model layer"):
        load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")
    with_manifest(lambda m: m["layers"][0].update(file="../layer_000.pt"))
    with pytest.raises(ValueError, match="local filenames"):
        load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")
    with_manifest(lambda m: m["layers"][1].update(sha256="0" * 64))
    with pytest.raises(ValueError, match="hash mismatch"):
        load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")
    with_manifest(lambda m: m["layers"][1].update(group_size=8))
    with pytest.raises(ValueError, match="does not match packed payload"):
        load_bundle(tmp_path, model, expected_model_id="tiny-olmoe")
