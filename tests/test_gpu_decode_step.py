"""End-to-end decode parity on the GPU: the captured step (native step engine and per-op engine)
against the CPU oracle on identical seeded weights and an identical prefilled cache.

Gates (the stated parity gates): weight codes and top-k expert ids bit-exact, logits KL < 1e-3 and
greedy tokens identical over the decode steps.
"""

from __future__ import annotations

import math
import os

import pytest
import torch

from gpu_util import (PER_KERNEL_REL_TOL, install_canonical, lemoq_model_from_oracle, oracle_state_from_session,
                      oracle_weights_from_model, rel_err)
from oracle import lemoq_oracle as ops
from oracle import olmoe_decode_oracle as glue

pytestmark = pytest.mark.gpu
DEV = "cuda"
KL_GATE = 1e-3


def _small_spec():
    return glue.OlmoeSpec(layers=2, hidden=256, heads=2, head_dim=128, experts=8, top_k=2, ffn=128, vocab=512)


def _small_whole_step_spec():
    """The smallest shape the whole-step kernel takes: every row width 512, head_dim 128."""
    return glue.OlmoeSpec(layers=2, hidden=512, heads=4, head_dim=128, experts=8, top_k=2, ffn=512, vocab=1024)


def _inject_oracle_cache(st):
    def hook(session):
        for i, cl in enumerate(session.cache.layers):
            cl.keys.copy_(st.keys[i].to(DEV))
            cl.values.copy_(st.values[i].to(DEV))
    return hook


def _fresh_oracle_state(spec, wq, prompt, max_len):
    st = glue.new_state(spec, max_len)
    first = glue.prefill(wq, st, prompt)
    return st, int(first.float().argmax())


def test_small_model_weights_prefill_and_decode_both_engines():
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits

    spec = _small_spec()
    ctx, new = 24, 8
    wf = glue.random_float_weights(spec, seed=3, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    # (1) quantised weights: codes and scales bit-exact against the oracle quantiser
    wg = oracle_weights_from_model(model, spec)
    for lo, lg in zip(wq.layers, wg.layers):
        assert torch.equal(lo.qkv_codes, lg.qkv_codes) and torch.equal(lo.qkv_scale, lg.qkv_scale)
        assert torch.equal(lo.o_codes, lg.o_codes) and torch.equal(lo.o_scale, lg.o_scale)
        assert torch.equal(lo.experts.packed_gate_up, lg.experts.packed_gate_up)
        assert torch.equal(lo.experts.scale_down, lg.experts.scale_down)
    assert torch.equal(wq.lm_head_codes, wg.lm_head_codes) and torch.equal(wq.lm_head_scale, wg.lm_head_scale)

    prompt = torch.tensor([[(7 * i + 3) % spec.vocab for i in range(ctx)]])
    st0, first_tok = _fresh_oracle_state(spec, wq, prompt[0], ctx + new)

    for engine in ("step", "ops"):
        session = StaticCacheDecodeSession(model, prompt.to(DEV), ctx=ctx, max_new_tokens=new, engine=engine)
        # (2) GPU eager prefill fills the cache like the oracle's prefill (fp16 matmul rounding apart)
        for i, cl in enumerate(session.cache.layers):
            assert rel_err(cl.keys[:, :, :ctx], st0.keys[i][:, :, :ctx]) < 2e-2
            assert rel_err(cl.values[:, :, :ctx], st0.values[i][:, :, :ctx]) < 2e-2
        assert session.seed_token_id == first_tok
        # (3) decode from the oracle's cache state: identical inputs on both sides
        session.after_prefill = _inject_oracle_cache(st0)
        session.capture(warmup=2)
        assert session.capture_info["engine"] == engine
        st = glue.new_state(spec, ctx + new)
        for i in range(spec.layers):
            st.keys[i].copy_(st0.keys[i])
            st.values[i].copy_(st0.values[i])
        glue.build_int8_mirror(st)
        session.reset()
        session.current_token_id = first_tok
        tok = first_tok
        ref_logits, got_logits, ref_tokens, got_tokens = [], [], [], []
        for s in range(new):
            trace = {}
            lg = glue.decode_step(wq, st, tok, ctx + s, kv_int8=True, trace=trace)
            session.replay(synchronize=True)
            got = session.logits_cpu().reshape(-1)
            ref_logits.append(lg)
            got_logits.append(got)
            tok = int(lg.float().argmax())
            ref_tokens.append(tok)
            got_tokens.append(session.current_token_id)
            if engine == "step":
                ids = session.step_topk_ids()
                for li in range(spec.layers):
                    assert ids[li].cpu().tolist() == trace["layers"][li]["top_i"].tolist(), (s, li)
            assert rel_err(got, lg) < 5 * PER_KERNEL_REL_TOL, (engine, s)
            assert got_tokens == ref_tokens, (engine, s)
        rep = compare_logits(ref_logits, got_logits)
        assert rep["kl"] < KL_GATE and rep["top1_agreement"] == 1.0, rep
        # the new K/V rows landed in the right slots of both caches
        for i, cl in enumerate(session.cache.layers):
            assert rel_err(cl.keys[:, :, ctx:ctx + new], st.keys[i][:, :, ctx:ctx + new]) < 2e-2
            bufs = model.model.layers[i].self_attn._lemoq_kv_int8_bufs
            diff = (bufs["kc"][:, :, ctx:ctx + new].cpu().int() - st.mirror[i]["kc"][:, :, ctx:ctx + new].int()).abs()
            assert int(diff.max()) <= 2 and float((diff == 0).float().mean()) > 0.97
            assert torch.equal(bufs["kc"][:, :, :ctx].cpu(), st.mirror[i]["kc"][:, :, :ctx])
            assert torch.isfinite(cl.keys).all()
        if engine == "step":
            assert session.step_error_flags() == 0
        # (4) graph replay == the same path run eagerly (bitwise: deterministic kernels)
        session.reset()
        session.current_token_id = first_tok
        eager = [session.decode_eager().float().cpu().reshape(-1).clone() for _ in range(new)]
        assert all(torch.equal(a, b.float()) for a, b in zip(eager, got_logits)), engine
        session.close()


def test_small_model_whole_step_kernel_odd_capacity():
    """The whole-step kernel on its smallest shape, with a cache capacity that is no multiple of the KV tile (or of
    anything): ids, tokens, logits and the new KV rows against the oracle from identical caches."""
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits

    spec = _small_whole_step_spec()
    ctx, new = 61, 6  # capacity 67: the last KV tile of every head is short and unaligned
    wf = glue.random_float_weights(spec, seed=5, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    prompt = torch.tensor([[(11 * i + 5) % spec.vocab for i in range(ctx)]])
    st, first_tok = _fresh_oracle_state(spec, wq, prompt[0], ctx + new)
    glue.build_int8_mirror(st)
    session = StaticCacheDecodeSession(model, prompt.to(DEV), ctx=ctx, max_new_tokens=new, engine="step")
    session.after_prefill = _inject_oracle_cache(st)
    session.capture(warmup=1)
    assert session.capture_info["kernels_per_step"] == 1 and session.capture_info["step_kernel"] == "whole-step"
    session.reset()
    session.current_token_id = first_tok
    tok = first_tok
    ref_logits, got_logits = [], []
    for s_ in range(new):
        trace = {}
        lg = glue.decode_step(wq, st, tok, ctx + s_, kv_int8=True, trace=trace)
        session.replay(synchronize=True)
        got = session.logits_cpu().reshape(-1)
        ids = session.step_topk_ids()
        for li in range(spec.layers):
            assert ids[li].cpu().tolist() == trace["layers"][li]["top_i"].tolist(), (s_, li)
        assert rel_err(got, lg) < 5 * PER_KERNEL_REL_TOL, s_
        tok = int(lg.float().argmax())
        assert session.current_token_id == tok, s_
        ref_logits.append(lg)
        got_logits.append(got)
    assert compare_logits(ref_logits, got_logits)["kl"] < KL_GATE
    assert session.step_error_flags() == 0
    for i, cl in enumerate(session.cache.layers):
        assert rel_err(cl.keys[:, :, ctx:ctx + new], st.keys[i][:, :, ctx:ctx + new]) < 2e-2
        bufs = model.model.layers[i].self_attn._lemoq_kv_int8_bufs
        assert torch.equal(bufs["kc"][:, :, :ctx].cpu(), st.mirror[i]["kc"][:, :, :ctx])
        assert torch.equal(bufs["vc"][:, :, :ctx].cpu(), st.mirror[i]["vc"][:, :, :ctx])
    session.close()


def test_small_model_fp16_kv_arm(monkeypatch):
    """kv_int8 switched off: the step attends to the fp16 cache (the reference's fp16-KV variant)."""
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits

    monkeypatch.setenv("LEMOQ_KV_INT8", "0")
    spec = _small_spec()
    ctx, new = 24, 6
    wf = glue.random_float_weights(spec, seed=4, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    prompt = torch.tensor([[(5 * i + 1) % spec.vocab for i in range(ctx)]])
    st, first_tok = _fresh_oracle_state(spec, wq, prompt[0], ctx + new)
    session = StaticCacheDecodeSession(model, prompt.to(DEV), ctx=ctx, max_new_tokens=new, engine="step")
    session.after_prefill = _inject_oracle_cache(st)
    session.capture(warmup=1)
    session.reset()
    session.current_token_id = first_tok
    toks, logits = glue.greedy_decode(wq, st, first_tok, ctx, new, kv_int8=False)
    got_logits, got_toks = [], []
    for _ in range(new):
        session.replay(synchronize=True)
        got_logits.append(session.logits_cpu().reshape(-1))
        got_toks.append(session.current_token_id)
    assert got_toks == toks
    assert compare_logits(logits, got_logits)["kl"] < KL_GATE
    session.close()


SHAPES = {
    # every row width 1024, expert rows of 2048 (one routed expert per down tile), renormalised routing weights
    "wide-ffn-renorm": dict(layers=2, hidden=1024, heads=8, head_dim=128, experts=16, top_k=4, ffn=2048, vocab=1000, norm_topk_prob=True),
    # 128 experts (four per lane in the routing warp), sixteen routed: the activation planes are at their 8192-value limit
    "many-experts": dict(layers=2, hidden=512, heads=4, head_dim=128, experts=128, top_k=16, ffn=512, vocab=1024),
    # one routed expert (no pairing of experts in a down tile), full hidden width, three layers
    "one-expert": dict(layers=3, hidden=2048, heads=16, head_dim=128, experts=8, top_k=1, ffn=1024, vocab=2048),
}


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_whole_step_kernel_other_shapes(shape):
    """Shapes at the corners of what the whole-step kernel takes, against the oracle from identical caches: tokens,
    logits, and the expert ids (exact against the oracle's routing of the step's OWN router logits)."""
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits

    spec = glue.OlmoeSpec(**SHAPES[shape])
    ctx, new = 70, 5
    wf = glue.random_float_weights(spec, seed=31, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    prompt = torch.tensor([[(17 * i + 3) % spec.vocab for i in range(ctx)]])
    st, first_tok = _fresh_oracle_state(spec, wq, prompt[0], ctx + new)
    glue.build_int8_mirror(st)
    session = StaticCacheDecodeSession(model, prompt.to(DEV), ctx=ctx, max_new_tokens=new, engine="step")
    session.after_prefill = _inject_oracle_cache(st)
    session.capture(warmup=1)
    assert session.capture_info["kernels_per_step"] == 1 and session.capture_info["step_kernel"] == "whole-step", shape
    session.reset()
    session.current_token_id = first_tok
    toks, logits = glue.greedy_decode(wq, st, first_tok, ctx, new, kv_int8=True)
    got_logits, got_toks = [], []
    for _ in range(new):
        session.replay(synchronize=True)
        got_logits.append(session.logits_cpu().reshape(-1))
        got_toks.append(session.current_token_id)
        ids, own = session.step_topk_ids().cpu(), session.step_router_logits().cpu()
        for li in range(spec.layers):
            _, want = ops.routing_softmax_topk(own[li:li + 1], spec.top_k, spec.norm_topk_prob)
            assert want.reshape(-1).tolist() == ids[li].tolist(), (shape, li)
    assert session.step_error_flags() == 0
    assert got_toks == toks, shape
    assert compare_logits(logits, got_logits)["kl"] < KL_GATE
    for s_, (ref, got) in enumerate(zip(logits, got_logits)):
        assert rel_err(got, ref) < 5 * PER_KERNEL_REL_TOL, (shape, s_)
    session.close()


def test_small_model_whole_step_kernel_fp16_kv_odd_capacity(monkeypatch):
    """The whole-step kernel attending to the fp16 cache (kv_int8 off): KV tiles of 32 positions, a capacity (67) that
    leaves the last tile of every head three rows long, the new token's row patched in from the block that wrote it."""
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits

    monkeypatch.setenv("LEMOQ_KV_INT8", "0")
    spec = _small_whole_step_spec()
    ctx, new = 61, 6
    wf = glue.random_float_weights(spec, seed=6, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    prompt = torch.tensor([[(11 * i + 5) % spec.vocab for i in range(ctx)]])
    st, first_tok = _fresh_oracle_state(spec, wq, prompt[0], ctx + new)
    session = StaticCacheDecodeSession(model, prompt.to(DEV), ctx=ctx, max_new_tokens=new, engine="step")
    session.after_prefill = _inject_oracle_cache(st)
    session.capture(warmup=1)
    assert session.capture_info["kernels_per_step"] == 1 and session.capture_info["step_kernel"] == "whole-step"
    session.reset()
    session.current_token_id = first_tok
    toks, logits = glue.greedy_decode(wq, st, first_tok, ctx, new, kv_int8=False)
    got_logits, got_toks = [], []
    for _ in range(new):
        session.replay(synchronize=True)
        got_logits.append(session.logits_cpu().reshape(-1))
        got_toks.append(session.current_token_id)
    assert session.step_error_flags() == 0
    assert got_toks == toks
    assert compare_logits(logits, got_logits)["kl"] < KL_GATE
    for s_, (ref, got) in enumerate(zip(logits, got_logits)):
        assert rel_err(got, ref) < 5 * PER_KERNEL_REL_TOL, s_
    # the rows the step wrote into the fp16 cache are the oracle's up to the rounding the activations carry
    for i, cl in enumerate(session.cache.layers):
        assert rel_err(cl.keys[:, :, ctx:ctx + new], st.keys[i][:, :, ctx:ctx + new]) < 2e-2, i
        assert rel_err(cl.values[:, :, ctx:ctx + new], st.values[i][:, :, ctx:ctx + new]) < 2e-2, i
    session.close()


@pytest.fixture
def whole_step_kernel():
    """The step engine as the single cooperative kernel (the default when the shapes allow it)."""
    from lemoq import _cabi

    _cabi.call("lemoq_set_tuning", 4, 1)
    yield
    _cabi.call("lemoq_set_tuning", 4, 1)


@pytest.fixture
def chained_kernels():
    """The step engine as chained per-op kernels with programmatic dependent launch (tuning key 4 = 0)."""
    from lemoq import _cabi

    _cabi.call("lemoq_set_tuning", 4, 0)
    yield
    _cabi.call("lemoq_set_tuning", 4, 1)


def test_one_full_size_layer_whole_step_kernel(whole_step_kernel):
    _one_full_size_layer(expect_kernels=1)


def test_one_full_size_layer_chained_kernels(chained_kernels):
    _one_full_size_layer(expect_kernels=None)


def test_one_full_size_layer_whole_step_kernel_ctx_4096(whole_step_kernel):
    """benchmark configuration 3's length: every warp of an attention block walks more than one block of positions."""
    _one_full_size_layer(expect_kernels=1, ctx=4096)


def _one_full_size_layer(expect_kernels, ctx=1024):
    """One OLMoE-sized decoder layer (hidden 2048, 16x128 heads, 64 experts top-8, ffn 1024) decoding at
    position 1024 over a seeded N(0,1) fp16 KV cache, input hidden N(0,1): logits, expert ids, KV codes."""
    from benchmarks.cudagraph import StaticCacheDecodeSession

    spec = glue.OlmoeSpec(layers=1, vocab=2048)
    new = 2
    wf = glue.random_float_weights(spec, seed=0, dtype=torch.float16, std=0.02)
    g = torch.Generator().manual_seed(1)
    wf.embed[7] = torch.randn(spec.hidden, generator=g).half()  # the input hidden state
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    st = glue.new_state(spec, ctx + new)
    st.keys[0][:, :, :ctx] = torch.randn(1, spec.heads, ctx, spec.head_dim, generator=g).half()
    st.values[0][:, :, :ctx] = torch.randn(1, spec.heads, ctx, spec.head_dim, generator=g).half()
    glue.build_int8_mirror(st)
    prompt = torch.full((1, ctx), 1, dtype=torch.long, device=DEV)
    results = {}
    for engine in ("step", "ops"):
        session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=new, engine=engine)
        session.after_prefill = _inject_oracle_cache(st)
        session.capture(warmup=1)
        session.reset()
        session.current_token_id = 7
        session.replay(synchronize=True)
        results[engine] = session.logits_cpu().reshape(-1)
        if engine == "step":
            # no data atomics anywhere: the same step from the same state gives the same bits
            session.reset()
            session.current_token_id = 7
            session.replay(synchronize=True)
            assert torch.equal(session.logits_cpu().reshape(-1), results[engine])
            ids = session.step_topk_ids()[0].cpu().tolist()
            assert session.step_error_flags() == 0
            if expect_kernels is not None:
                assert session.capture_info["kernels_per_step"] == expect_kernels
        bufs = model.model.layers[0].self_attn._lemoq_kv_int8_bufs
        kc_new, ks_new = bufs["kc"][0, :, ctx].cpu(), bufs["ks"][0, :, ctx].cpu()
        k_new = session.cache.layers[0].keys[0, :, ctx].cpu()
        session.close()
        # the int8 row written by the step is exactly the quantisation of the fp16 row it wrote
        rc, rs = ops.kv_quantize_per_token(k_new)
        assert torch.equal(kc_new, rc) and torch.equal(ks_new, rs)
    trace = {}
    ref = glue.decode_step(wq, st, 7, ctx, kv_int8=True, trace=trace)
    assert ids == trace["layers"][0]["top_i"].tolist()
    for engine, got in results.items():
        assert rel_err(got, ref) < 2 * PER_KERNEL_REL_TOL, engine
        assert int(got.float().argmax()) == int(ref.float().argmax())
    assert rel_err(k_new, st.keys[0][0, :, ctx]) < PER_KERNEL_REL_TOL


def test_full_model_whole_step_kernel(whole_step_kernel):
    _full_model_greedy(1024, expect_kernels=1)


def test_full_model_chained_kernels(chained_kernels):
    _full_model_greedy(1024, expect_kernels=None)


def test_full_model_whole_step_kernel_ctx_4096(whole_step_kernel):
    """Benchmark configuration 3: the canonical cell at ctx 4096."""
    _full_model_greedy(4096, expect_kernels=1)


def test_full_model_fp16_kv_arm_ctx_4096(whole_step_kernel, monkeypatch):
    """Benchmark configuration 3's comparison arm: the same model attending to the fp16 cache (kv_int8 off), as one
    kernel per step."""
    monkeypatch.setenv("LEMOQ_KV_INT8", "0")
    _full_model_greedy(4096, expect_kernels=1, kv_int8=False, steps=16)


def test_full_model_fp16_kv_arm_ctx_4096_chained_kernels(chained_kernels, monkeypatch):
    monkeypatch.setenv("LEMOQ_KV_INT8", "0")
    _full_model_greedy(4096, expect_kernels=None, kv_int8=False, steps=8)


def _full_model_greedy(ctx, expect_kernels, kv_int8=True, steps=32):
    """The canonical cell at full size: 16 layers, vocab 50304, all-ones prompt prefilled on the GPU,
    then 32 greedy steps through the captured graph; the oracle decodes on the CPU from a copy of the
    same prefilled cache with the same quantised weights."""
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits
    from benchmarks.runner import build_model

    spec = glue.OlmoeSpec()
    model = build_model(seed=0)
    install_canonical(model, ctx, steps)
    prompt = torch.full((1, ctx), 1, dtype=torch.long, device=DEV)
    session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=steps, engine="step")
    session.capture(warmup=3)
    if expect_kernels is not None:
        assert session.capture_info["kernels_per_step"] == expect_kernels
    session.reset()
    first = session.seed_token_id
    wq = oracle_weights_from_model(model, spec)
    st = oracle_state_from_session(session, spec)
    got_logits, got_toks, got_ids = [], [], []
    for _ in range(steps):
        session.replay(synchronize=True)
        got_logits.append(session.logits_cpu().reshape(-1))
        got_toks.append(session.current_token_id)
        got_ids.append(session.step_topk_ids().cpu())
        # the routing is bit-exact on ITS OWN inputs: the oracle's softmax/top-k of the step's router logits gives the
        # step's expert ids, order included (so a flip against the oracle's ids below can only come from the logits)
        own = session.step_router_logits().cpu()
        for li in range(spec.layers):
            _, want = ops.routing_softmax_topk(own[li:li + 1], spec.top_k, spec.norm_topk_prob)
            assert want.reshape(-1).tolist() == got_ids[-1][li].tolist(), (len(got_ids) - 1, li)
    assert session.step_error_flags() == 0
    session.close()
    del model
    torch.cuda.empty_cache()
    tok = first
    ref_logits, ref_toks = [], []
    id_match = 0
    pair_match, pairs = 0, 0
    mismatches = []  # (step, layer, gap between the oracle's k-th and (k+1)-th router logit in fp16 ulps)
    for s in range(steps):
        trace = {}
        lg = glue.decode_step(wq, st, tok, ctx + s, kv_int8=kv_int8, trace=trace)
        ref_logits.append(lg)
        tok = int(lg.float().argmax())
        ref_toks.append(tok)
        ref_ids = torch.stack([t["top_i"] for t in trace["layers"]])
        same = (torch.sort(ref_ids, dim=1).values == torch.sort(got_ids[s], dim=1).values).all(dim=1)
        for li in (~same).nonzero().flatten().tolist():
            top = torch.sort(trace["layers"][li]["router_logits"].float().flatten(), descending=True).values
            ulp = 2.0 ** (math.floor(math.log2(max(abs(float(top[spec.top_k - 1])), 2.0 ** -14))) - 10)
            mismatches.append((s, li, float(top[spec.top_k - 1] - top[spec.top_k]) / ulp))
        id_match += int(same.all())
        pair_match += int(same.sum())
        pairs += int(same.numel())
    rep = compare_logits(ref_logits, got_logits)
    assert got_toks == ref_toks, (got_toks, ref_toks)
    assert rep["kl"] < KL_GATE and rep["top1_agreement"] == 1.0, rep
    # Expert sets on identical inputs are bit-exact (kernel-level tests).  End to end the inputs of a
    # router differ from the oracle's in the last fp16 bit now and then, and with random-init weights the
    # router logits are nearly flat, so the 8th/9th expert can swap: require >= 98 % of the (step, layer)
    # routings identical and most steps identical in every layer; KL and tokens above bound the effect.
    assert pair_match >= 0.98 * pairs, (pair_match, pairs, mismatches)
    # a differing expert set comes from a near tie at the top-k boundary of the oracle's logits (recorded above in
    # fp16 ulps; the step's own logits differ from the oracle's by rounding that has accumulated over layers and steps)
    assert all(gap_ulps <= 64.0 for _, _, gap_ulps in mismatches), mismatches
    assert id_match >= steps // 2, id_match


@pytest.mark.parametrize("whole", [True, False])
def test_chained_replays_equal_host_driven_replays(whole):
    """K replays with no host work in between (the step feeds itself: its pick, the next slot and the next length go
    into its own input scalars) give the tokens of K rounds of set-inputs / replay / read-back, token for token."""
    from benchmarks.cudagraph import StaticCacheDecodeSession
    from lemoq import _cabi

    _cabi.call("lemoq_set_tuning", 4, 1 if whole else 0)
    try:
        spec = _small_whole_step_spec()
        ctx, new = 40, 24
        wf = glue.random_float_weights(spec, seed=9, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
        model = lemoq_model_from_oracle(wf)
        install_canonical(model, ctx, new)
        prompt = torch.tensor([[(13 * i + 1) % spec.vocab for i in range(ctx)]], device=DEV)
        session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=new, engine="step")
        session.capture(warmup=1)
        assert (session.capture_info["kernels_per_step"] == 1) == whole
        session.reset()
        host_driven, host_logits = [], None
        for _ in range(new):
            session.replay(synchronize=True)
            host_driven.append(session.current_token_id)
        host_logits = session.logits_cpu().clone()
        session.reset()
        chained = session.replay_chained(10) + session.replay_chained(new - 10)
        assert chained == host_driven
        assert session.position == ctx + new and session.current_token_id == host_driven[-1]
        assert torch.equal(session.logits_cpu(), host_logits)
        assert session.step_error_flags() == 0
        with pytest.raises(RuntimeError, match="exceeded StaticCache capacity"):
            session.replay_chained(1)
        session.close()
    finally:
        _cabi.call("lemoq_set_tuning", 4, 1)


@pytest.mark.parametrize("whole", [True, False])
def test_out_of_range_step_scalars_raise_flags_instead_of_faulting(whole):
    """A position / length beyond the cache capacity is clamped by the kernels and reported through the flag
    word (LEMOQ_FLAG_BAD_POSITION = 1, LEMOQ_FLAG_BAD_LENGTH = 2); nothing is written outside the caches."""
    from benchmarks.cudagraph import StaticCacheDecodeSession
    from lemoq import _cabi

    _cabi.call("lemoq_set_tuning", 4, 1 if whole else 0)
    try:
        spec = glue.OlmoeSpec(layers=1, vocab=2048)
        ctx, new = 64, 2
        wf = glue.random_float_weights(spec, seed=2, dtype=torch.float16, std=0.02)
        model = lemoq_model_from_oracle(wf)
        install_canonical(model, ctx, new)
        prompt = torch.full((1, ctx), 1, dtype=torch.long, device=DEV)
        session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=new, engine="step")
        session.capture(warmup=1)
        assert session.capture_info["kernels_per_step"] == (1 if whole else session.capture_info["kernels_per_step"])
        session.reset()
        session.replay(synchronize=True)
        assert session.step_error_flags() == 0
        before = [cl.keys.clone() for cl in session.cache.layers]
        cap = session.config.max_cache_len
        session.buffers.cache_position.fill_(cap + 5)
        session.buffers.filled_len.fill_(cap + 7)
        with torch.cuda.stream(session.stream):
            session.graph.replay()
        session.stream.synchronize()
        assert session.step_error_flags() == 1 | 2
        assert torch.isfinite(session.logits.float()).all()
        for cl, b in zip(session.cache.layers, before):
            assert torch.equal(cl.keys, b)  # the out-of-range row was not written anywhere
        # a token id outside the vocabulary is clamped too (LEMOQ_FLAG_BAD_TOKEN = 16) instead of reading past the table
        session.reset()
        session.buffers.token.fill_(spec.vocab + 12345)
        with torch.cuda.stream(session.stream):
            session.graph.replay()
        session.stream.synchronize()
        assert session.step_error_flags() & 16
        assert torch.isfinite(session.logits.float()).all()
        assert 0 <= int(session.step_next_token.item()) < spec.vocab
        session.close()
    finally:
        _cabi.call("lemoq_set_tuning", 4, 1)


def test_a_wait_that_runs_out_raises_the_flag_and_the_next_step_is_unaffected():
    """The time-out path of the whole-step kernel's flagged-word waits, exercised without anything hanging: with the
    poll limit at 1 (tuning key 5) a reader gives up on the first look, the step goes on with stale values, returns,
    and reports LEMOQ_FLAG_WAIT_TIMEOUT (8).  Every copy is still awaited and every index still comes from clamped
    scalars or lane numbers, so nothing but the values is affected; with the limit restored the same session decodes
    the same tokens as before."""
    from benchmarks.cudagraph import StaticCacheDecodeSession
    from lemoq import _cabi

    spec = _small_whole_step_spec()
    ctx, new = 40, 6
    wf = glue.random_float_weights(spec, seed=13, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new)
    prompt = torch.tensor([[(3 * i + 7) % spec.vocab for i in range(ctx)]], device=DEV)
    session = StaticCacheDecodeSession(model, prompt, ctx=ctx, max_new_tokens=new, engine="step")
    session.capture(warmup=1)
    assert session.capture_info["step_kernel"] == "whole-step"

    def decode():
        session.reset()
        out = []
        for _ in range(new):
            session.replay(synchronize=True)
            out.append(session.current_token_id)
        return out

    good = decode()
    assert session.step_error_flags() == 0
    try:
        _cabi.call("lemoq_set_tuning", 5, 1)
        session.reset()
        session.replay(synchronize=True)  # returns: the waits are bounded
        assert session.step_error_flags() & 8
        assert 0 <= session.current_token_id < spec.vocab  # the pick is a valid id whatever the logits are
    finally:
        _cabi.call("lemoq_set_tuning", 5, 1 << 21)
    session.clear_step_error_flags()
    assert decode() == good
    assert session.step_error_flags() == 0
    session.close()
