"""Batched lockstep decode (the expert-parallel mode at world size 1) against the CPU oracle decoding each
sequence on its own: same quantised weights, the same prefilled cache, distinct first tokens.  The
multi-rank exchange itself is covered on the CPU (two gloo ranks) and, on a multi-GPU box, by comparing
the tokens of `benchmarks/expert_parallel.py` at G ranks with its own output at one rank."""

from __future__ import annotations

import pytest
import torch

from gpu_util import install_canonical, lemoq_model_from_oracle
from oracle import olmoe_decode_oracle as glue

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_batched_lockstep_decode_matches_oracle_per_sequence():
    from benchmarks.cudagraph import StaticCacheDecodeSession, compare_logits
    from benchmarks.expert_parallel import ExpertParallelDecoder

    spec = glue.OlmoeSpec(layers=2, hidden=256, heads=2, head_dim=128, experts=8, top_k=2, ffn=128, vocab=512)
    ctx, new, seqs = 24, 5, 3
    wf = glue.random_float_weights(spec, seed=11, dtype=torch.float16, std=0.05, norm_weight_jitter=0.1)
    wq = glue.quantize_weights(wf)
    model = lemoq_model_from_oracle(wf)
    install_canonical(model, ctx, new + 2)
    prompt = torch.tensor([[(7 * i + 3) % spec.vocab for i in range(ctx)]])
    st0 = glue.new_state(spec, ctx + new + 2)
    glue.prefill(wq, st0, prompt[0])
    session = StaticCacheDecodeSession(model, prompt.to(DEV), ctx=ctx, max_new_tokens=new + 2, engine="ops")
    for i, cl in enumerate(session.cache.layers):  # identical inputs on both sides: the oracle's prefilled cache
        cl.keys.copy_(st0.keys[i].to(DEV))
        cl.values.copy_(st0.values[i].to(DEV))
    dec = ExpertParallelDecoder(model, session, sequences=seqs, world=1, rank=0, attn_splits=3)
    first = [5, 77, 300]
    tokens = torch.tensor(first, dtype=torch.int64, device=DEV)
    got_logits, got_tokens = [], []
    for _ in range(new):
        lg = dec.step(tokens)
        tokens = lg.float().argmax(dim=-1)
        got_logits.append(lg.float().cpu())
        got_tokens.append(tokens.cpu())
    assert dec.error_flags() == 0
    for s, tok0 in enumerate(first):
        st = glue.new_state(spec, ctx + new + 2)
        for i in range(spec.layers):
            st.keys[i].copy_(st0.keys[i])
            st.values[i].copy_(st0.values[i])
        glue.build_int8_mirror(st)
        ref_tokens, ref_logits = glue.greedy_decode(wq, st, tok0, ctx, new, kv_int8=True)
        assert [int(t[s]) for t in got_tokens] == ref_tokens, s
        rep = compare_logits(ref_logits, [g[s] for g in got_logits])
        assert rep["kl"] < 1e-3 and rep["top1_agreement"] == 1.0, (s, rep)
