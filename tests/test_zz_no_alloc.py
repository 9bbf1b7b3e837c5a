"""The int8 decode attention entry point that takes no workspace (its scratch is a fixed array inside the
library) against the workspace-taking entry point, through the C ABI.  Collected last on purpose: it must
pass on its own and after every other GPU test has used the library."""

from __future__ import annotations

import math

import pytest
import torch

from gpu_util import PER_KERNEL_REL_TOL, rel_err
from oracle import lemoq_oracle as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(heads, seq, dim, filled, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(heads, dim, generator=g).half().to(DEV)
    kc = torch.randint(-127, 128, (heads, seq, dim), generator=g, dtype=torch.int8).to(DEV)
    vc = torch.randint(-127, 128, (heads, seq, dim), generator=g, dtype=torch.int8).to(DEV)
    ks = (torch.rand(heads, seq, generator=g) * 0.02 + 0.001).half().to(DEV)
    vs = (torch.rand(heads, seq, generator=g) * 0.02 + 0.001).half().to(DEV)
    fl = torch.tensor([filled], dtype=torch.int32, device=DEV)
    return q, kc, ks, vc, vs, fl


def _with_workspace(case, heads, seq, dim, splits):
    from lemoq import _cabi

    q, kc, ks, vc, vs, fl = case
    ws = torch.zeros(int(_cabi.lib().lemoq_attn_workspace_bytes(heads, dim, splits)), dtype=torch.uint8, device=DEV)
    out = torch.empty(heads, dim, dtype=torch.float16, device=DEV)
    _cabi.call("lemoq_attn_decode_int8", _cabi.ptr(q), _cabi.ptr(kc), _cabi.ptr(ks), _cabi.ptr(vc), _cabi.ptr(vs), seq * dim,
               _cabi.ptr(fl), _cabi.ptr(out), heads, seq, dim, splits, 1.0 / math.sqrt(dim), _cabi.ptr(ws), None,
               _cabi.current_stream(q.device))
    torch.cuda.synchronize()
    return out


def _static(case, heads, seq, dim, splits):
    from lemoq import _cabi

    q, kc, ks, vc, vs, fl = case
    out = torch.empty(heads, dim, dtype=torch.float16, device=DEV)
    _cabi.call("lemoq_attn_decode_int8_static", _cabi.ptr(q), _cabi.ptr(kc), _cabi.ptr(ks), _cabi.ptr(vc), _cabi.ptr(vs),
               seq * dim, _cabi.ptr(fl), _cabi.ptr(out), heads, seq, dim, splits, 1.0 / math.sqrt(dim), None,
               _cabi.current_stream(q.device))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("heads,seq,dim,filled,splits", [(16, 1024, 128, 1000, 9), (4, 300, 64, 257, 5)])
def test_static_scratch_matches_workspace_entry_twice_in_a_row(heads, seq, dim, filled, splits):
    case = _case(heads, seq, dim, filled, seed=heads + seq)
    ref = _with_workspace(case, heads, seq, dim, splits)
    first = _static(case, heads, seq, dim, splits)
    second = _static(case, heads, seq, dim, splits)  # the shared array must have been left ready for the next call
    assert torch.isfinite(first.float()).all()
    assert torch.equal(first, ref)  # same kernel, same layout of the partials: the same bits
    assert torch.equal(first, second)
    assert rel_err(first, _oracle(case, filled, dim)) < PER_KERNEL_REL_TOL
    # a different shape right after reuses the same array
    case2 = _case(8, 512, 128, 512, seed=5)
    assert rel_err(_static(case2, 8, 512, 128, 3), _with_workspace(case2, 8, 512, 128, 3)) < PER_KERNEL_REL_TOL


def _oracle(case, filled, dim):
    q, kc, ks, vc, vs, _ = case
    return ops.attention_int8(q.cpu(), kc.cpu(), ks.cpu(), vc.cpu(), vs.cpu(), filled, scale=1.0 / math.sqrt(dim))


def test_static_scratch_shapes_of_different_head_counts_share_the_array():
    """A call with few heads leaves partials where a layout sized per call would put the counters of a
    later call with more heads: the counters sit in a fixed region, so the second shape is still right.
    Also: a call allocates nothing (the free device memory does not move)."""
    small = _case(16, 256, 128, 256, seed=11)
    assert rel_err(_static(small, 16, 256, 128, 4), _oracle(small, 256, 128)) < PER_KERNEL_REL_TOL
    heads, seq, dim, filled, splits = 80, 192, 64, 150, 2
    big = _case(heads, seq, dim, filled, seed=12)
    free_before = torch.cuda.mem_get_info()[0]
    got = _static(big, heads, seq, dim, splits)
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.isfinite(got.float()).all()
    assert rel_err(got, _oracle(big, filled, dim)) < PER_KERNEL_REL_TOL
    assert torch.equal(got, _with_workspace(big, heads, seq, dim, splits))
    again = _static(small, 16, 256, 128, 4)
    assert rel_err(again, _oracle(small, 256, 128)) < PER_KERNEL_REL_TOL
    # just under the array's size: 16 KiB of counters + 63 * 31 * 130 * 4 bytes of partials
    edge = _case(63, 64, 128, 64, seed=13)
    assert rel_err(_static(edge, 63, 64, 128, 31), _oracle(edge, 64, 128)) < PER_KERNEL_REL_TOL


def test_static_scratch_refuses_sizes_beyond_its_maximum():
    from lemoq import _cabi

    limit = int(_cabi.lib().lemoq_attn_static_scratch_bytes())
    assert limit == 1 << 20
    heads, seq, dim, splits = 16, 64, 128, 4096  # 16 * 4096 * 130 * 4 bytes = 34 MB of partials
    case = _case(heads, seq, dim, 64, seed=1)
    with pytest.raises(ValueError, match="fixed array"):
        _static(case, heads, seq, dim, splits)
