"""The int8 decode attention entry point that takes no workspace (its scratch is a fixed array inside the
library) against the workspace-taking entry point, through the C ABI.  Collected last on purpose: it must
pass on its own and after every other GPU test has used the library."""

from __future__ import annotations

import math

import pytest
import torch

from gpu_util import PER_KERNEL_REL_TOL, rel_err

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
    assert rel_err(first, ref) < PER_KERNEL_REL_TOL
    assert rel_err(second, ref) < PER_KERNEL_REL_TOL
    assert torch.equal(first, second)
    # a different shape right after reuses the same array
    case2 = _case(8, 512, 128, 512, seed=5)
    assert rel_err(_static(case2, 8, 512, 128, 3), _with_workspace(case2, 8, 512, 128, 3)) < PER_KERNEL_REL_TOL


def test_static_scratch_refuses_sizes_beyond_its_maximum():
    from lemoq import _cabi

    limit = int(_cabi.lib().lemoq_attn_static_scratch_bytes())
    assert limit == 1 << 20
    heads, seq, dim, splits = 16, 64, 128, 4096  # 16 * 4096 * 130 * 4 bytes = 34 MB of partials
    case = _case(heads, seq, dim, 64, seed=1)
    with pytest.raises(ValueError, match="fixed array"):
        _static(case, heads, seq, dim, splits)
