"""The runner's GPU path (reference: benchmarks/runner.py:1067-1348): install order, capture, the graph-vs-eager
correctness gate (benchmarks/runner.py:1237-1273), timing (benchmarks/cudagraph.py:420-495) and the payload."""

from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu

CANONICAL = {"bit_width": "w8a16", "dequant": "fused", "group_size": 128}


@pytest.mark.parametrize("engine", ["step", "ops"])
def test_run_cudagraph_two_layers(engine):
    from benchmarks.runner import run_cudagraph

    payload = run_cudagraph(ctx=64, max_new_tokens=32, warmup=5, timed=20, attn="kernel", moe="grouped", quant_cfg=CANONICAL,
                            rmsnorm="fused", layers=2, seed=0, engine=engine, bandwidth_gbs=6552.0)
    assert payload["status"] == "measured"
    cfg = payload["config"]
    assert cfg["execution"] == "cudagraph" and cfg["attn"] == "kernel" and cfg["moe"] == "grouped" and cfg["layers"] == 2
    for switch in ("fused_rope", "fused_route", "skip_mask_fill", "packed_qkv", "kv_direct_write", "lm_head_w8", "kv_int8"):
        assert any(switch in key for key in cfg), (switch, sorted(cfg))
    # the gate: graph replay against the same path run eagerly from the same prefilled state
    gate = payload["correctness"]
    assert gate["passed"] and gate["token_sequence_match"] and gate["seed_token_match"]
    assert gate["kl"] <= 1e-5 and gate["top1_agreement"] == 1.0 and gate["steps"] == 32 and len(gate["tokens"]) == 32
    cap = payload["capture"]
    assert cap["engine"] == engine and cap["replay_success"]
    if engine == "step":
        assert cap["kernels_per_step"] == 1 and cap["step_kernel"] == "whole-step"
    install = payload["install"]
    assert install["attn_replaced"] == 2 and install["moe_replaced"] == 2 and install["packed_qkv_modules"] == 2
    timing = payload["timing"]
    assert timing["status"] == "measured" and timing["wall_p50_ms"] > 0 and timing["gpu_busy_ms"] > 0
    assert timing["gpu_busy_ms"] <= timing["wall_p50_ms"] * 1.5
    assert payload["bytes"]["T"] == payload["bytes"]["W"] + payload["bytes"]["KV"]
    assert payload["ms_per_token"] == timing["wall_p50_ms"]
    assert 0.0 < payload["floor_fraction_gpu"] < 1.5


def test_run_cudagraph_refuses_a_horizon_shorter_than_the_timed_window():
    from benchmarks.runner import check_refusals

    with pytest.raises(ValueError, match="timed"):
        check_refusals(ctx=64, batch=1, execution="cudagraph", attn="kernel", moe="grouped", bit_width="w8a16", dequant="fused",
                       group_size=128, rmsnorm="fused", max_new_tokens=8, timed=20)
