"""Host logic of the batched expert-parallel decode: dispatch plan, variable-count all-to-all and the
slot-order combine, run as two gloo ranks on the CPU with a stand-in expert function.  The result of every
rank must equal what the same tokens give without any exchange, bit for bit."""

from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [p for p in (os.path.join(ROOT, "leanmoe-quant_b200"),) if p not in sys.path]

EXPERTS, TOP_K, HIDDEN = 8, 3, 16


def _fake_expert(x, global_ids):
    """Stand-in for an expert: a different fixed map per expert, rounded to fp16 like the kernels' output."""
    return (x.float() * (global_ids.float() + 1.0).unsqueeze(1) + global_ids.float().unsqueeze(1)).half()


def _inputs(rank, tokens):
    g = torch.Generator().manual_seed(100 + rank)
    h = torch.randn(tokens, HIDDEN, generator=g).half()
    top_i = torch.stack([torch.randperm(EXPERTS, generator=g)[:TOP_K] for _ in range(tokens)]).to(torch.int64)
    if rank == 1:
        top_i[:] = torch.tensor([0, 1, 2])  # one rank sends nothing at all to the other: zero-count splits
    top_w = torch.rand(tokens, TOP_K, generator=g).half()
    return h, top_w, top_i


def _expected(h, top_w, top_i):
    t, k = top_i.shape
    pairs = _fake_expert(h.repeat_interleave(k, dim=0), top_i.reshape(-1)).reshape(t, k, -1)
    return (pairs.float() * top_w.reshape(t, k, 1).float()).sum(dim=1).half()


def _worker(rank, world, port, tokens, static, failures):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from benchmarks.expert_parallel import expert_parallel_moe, expert_parallel_moe_static, plan_dispatch

        epr = EXPERTS // world
        h, top_w, top_i = _inputs(rank, tokens)
        seen = []

        def expert_fn(x, local_ids):
            assert torch.equal(local_ids, torch.sort(local_ids).values)       # grouped by expert
            seen.append(int(x.shape[0]))
            if static:
                # padding slots carry the id `epr` behind the real pairs; their outputs must never be used
                assert int(local_ids.min()) >= 0 and int(local_ids.max()) <= epr and x.shape[0] == world * tokens * TOP_K
                y = _fake_expert(x, local_ids + rank * epr)
                y[local_ids == epr] = float("nan")
                return y
            assert int(local_ids.min()) >= 0 and int(local_ids.max()) < epr  # only experts this rank owns arrive
            return _fake_expert(x, local_ids + rank * epr)

        moe = expert_parallel_moe_static if static else expert_parallel_moe
        out = moe(h, top_w, top_i, experts=EXPERTS, world=world, rank=rank, expert_fn=expert_fn)
        if not torch.equal(out, _expected(h, top_w, top_i)):
            failures.put((rank, "combined output differs from the exchange-free result"))
        plan = plan_dispatch(top_i, experts=EXPERTS, world=world)
        total = torch.tensor([sum(plan.send_counts), sum(plan.recv_counts)])
        dist.all_reduce(total)
        if int(total[0]) != int(total[1]) or sum(plan.send_counts) != tokens * TOP_K:
            failures.put((rank, "pair counts do not balance: %s" % (total.tolist(),)))
        if world > 1 and rank == 1 and plan.send_counts[1] != 0:
            failures.put((rank, "expected a zero-count split"))
    except Exception as exc:  # noqa: BLE001 - reported to the parent
        failures.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,tokens,static", [(2, 5, False), (1, 4, False), (2, 5, True), (1, 4, True)])
def test_dispatch_combine_matches_exchange_free_result(world, tokens, static):
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tokens, static, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0, "rank exited with %s" % p.exitcode
    errors = []
    while not failures.empty():
        errors.append(failures.get())
    assert not errors, errors


def test_plan_rejects_bad_shapes():
    from benchmarks.expert_parallel import plan_dispatch

    with pytest.raises(ValueError):
        plan_dispatch(torch.zeros(2, 2, dtype=torch.int64), experts=7, world=2)
    with pytest.raises(ValueError):
        plan_dispatch(torch.full((2, 2), 9, dtype=torch.int64), experts=8, world=1)
