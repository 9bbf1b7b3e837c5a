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


@pytest.mark.parametrize("exchange", ["dynamic", "static-tensor-library", "static-kernels"])
def test_batched_lockstep_decode_matches_oracle_per_sequence(exchange):
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
    dec = ExpertParallelDecoder(model, session, sequences=seqs, world=1, rank=0, attn_splits=3,
                                static_exchange=exchange != "dynamic", exchange_kernels=exchange == "static-kernels")
    assert dec.exchange_kernels == (exchange == "static-kernels")
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


def test_exchange_kernels_place_every_row_like_the_tensor_library_form():
    """Two ranks emulated on one GPU: each rank's dispatch, the blocks swapped by hand as the all-to-all would, regroup,
    a stand-in expert function that marks every row with its expert, give back, swap, combine - against the same steps
    of the tensor-library form (which the two-rank gloo test covers) and against the direct sum."""
    from lemoq import _cabi

    world, experts, t, k, hidden = 2, 8, 5, 3, 64
    epr, pairs = experts // world, t * k
    g = torch.Generator().manual_seed(5)
    h = [torch.randn(t, hidden, generator=g).half().to(DEV) for _ in range(world)]
    top_i = [torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(t)]).to(DEV) for _ in range(world)]
    top_i[0][0, 0] = top_i[0][1, 0]  # equal experts in different tokens: the stable order matters
    top_w = [torch.rand(t, k, generator=g).half().to(DEV) for _ in range(world)]
    stream = _cabi.current_stream(torch.device(DEV))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    send, slot = [], []
    for r in range(world):
        sb = torch.empty((world, pairs, hidden + 8), dtype=torch.float16, device=DEV)
        sl = torch.empty(pairs, dtype=torch.int32, device=DEV)
        src = torch.empty(world * pairs, dtype=torch.int32, device=DEV)
        _cabi.call("lemoq_ep_dispatch", _cabi.ptr(h[r]), _cabi.ptr(top_i[r]), t, k, hidden, experts, world, _cabi.ptr(sb), _cabi.ptr(sl),
                   _cabi.ptr(src), _cabi.ptr(err), stream)
        send.append(sb)
        slot.append(sl)
        # every pair sits where the stable sort by expert puts it, with its id behind the activations
        flat = top_i[r].reshape(-1)
        order = torch.argsort(flat, stable=True)
        dest = torch.div(flat[order], epr, rounding_mode="floor")
        counts = torch.bincount(dest, minlength=world)
        pos = torch.arange(pairs, device=DEV) - (torch.cumsum(counts, 0) - counts)[dest]
        assert torch.equal(sl[order].long(), dest * pairs + pos)
        assert torch.equal(sb[dest, pos, :hidden], h[r][torch.div(order, k, rounding_mode="floor")])
        assert torch.equal(sb[dest, pos, hidden].long(), flat[order])
        used = torch.zeros(world * pairs, dtype=torch.bool, device=DEV)
        used[sl.long()] = True
        assert bool((sb.reshape(-1, hidden + 8)[~used][:, hidden] == experts).all())
    back_blocks = [[None] * world for _ in range(world)]
    for r in range(world):  # what rank r receives: block r of every rank's send buffer
        recv = torch.stack([send[s][r] for s in range(world)]).contiguous()
        rows = world * pairs
        xs = torch.empty((rows, hidden), dtype=torch.float16, device=DEV)
        perm = torch.empty(rows, dtype=torch.int32, device=DEV)
        seg = torch.empty(epr + 1, dtype=torch.int32, device=DEV)
        _cabi.call("lemoq_ep_regroup", _cabi.ptr(recv), rows, hidden, experts, world, r, _cabi.ptr(xs), _cabi.ptr(perm), _cabi.ptr(seg),
                   _cabi.ptr(err), stream)
        ids = recv[:, :, hidden].reshape(-1).long()
        local = torch.where(ids == experts, torch.full_like(ids, epr), ids - r * epr)
        ref_perm = torch.argsort(local, stable=True)
        real = int((local < epr).sum())
        assert torch.equal(perm.long(), ref_perm)
        assert seg.tolist() == [int((local < e).sum()) for e in range(epr + 1)] and seg[-1] == real
        assert torch.equal(xs[:real], recv.reshape(-1, hidden + 8)[ref_perm[:real], :hidden]) and not bool(xs[real:].any())
        # stand-in experts: row of local expert l on rank r -> x * (r * epr + l + 1)
        ys = torch.full_like(xs, float("nan"))
        for e in range(epr):
            ys[seg[e]:seg[e + 1]] = xs[seg[e]:seg[e + 1]] * float(r * epr + e + 1)
        y = torch.zeros((world, pairs, hidden), dtype=torch.float16, device=DEV)
        _cabi.call("lemoq_ep_return", _cabi.ptr(ys), _cabi.ptr(perm), _cabi.ptr(seg), rows, hidden, epr, _cabi.ptr(y), stream)
        for s in range(world):
            back_blocks[s][r] = y[s]
    for r in range(world):
        back = torch.stack(back_blocks[r]).contiguous()
        out = torch.empty((t, hidden), dtype=torch.float16, device=DEV)
        _cabi.call("lemoq_ep_combine", _cabi.ptr(back), _cabi.ptr(slot[r]), _cabi.ptr(top_w[r]), t, k, hidden, _cabi.ptr(out), stream)
        per_pair = (h[r].unsqueeze(1) * (top_i[r] + 1).unsqueeze(-1).half()).float()  # the stand-in expert, rounded to fp16 like y
        ref = torch.zeros((t, hidden), dtype=torch.float32, device=DEV)
        for j in range(k):  # slot order, products and sums in fp32
            ref = ref + per_pair[:, j] * top_w[r][:, j].float().unsqueeze(-1)
        assert torch.equal(out, ref.half())
    assert int(err.item()) == 0
