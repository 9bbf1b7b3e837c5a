"""The weights-stationary W8 kernels for many tokens per call against the CPU oracle (per token / per pair):
dense rows, grouped experts with segments (an expert without tokens included), gate/up SwiGLU epilogue."""

from __future__ import annotations

import pytest
import torch

from gpu_util import PER_KERNEL_REL_TOL, rel_err
from oracle import lemoq_oracle as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


# K = 128 and 256: a token's planes and scales are not a multiple of 16 bytes by themselves
@pytest.mark.parametrize("tokens,n,k", [(13, 96, 2048), (1, 64, 512), (64, 258, 1024), (5, 64, 256), (3, 32, 128)])
def test_dense_rows_many_tokens(tokens, n, k):
    from lemoq.kernels.batched_w8 import w8_linear_tokens

    g = torch.Generator().manual_seed(tokens + n)
    w = torch.randn(n, k, generator=g) * 0.02
    codes, scale = ops.rtn_quantize_w8(w, 128)
    x = torch.randn(tokens, k, generator=g).half()
    x[0, :16] = 0  # an all-zero chunk
    x[-1, 5] = 30000.0  # a chunk with a huge dynamic range
    ref = ops.dense_w8_gemv(x, codes, scale, 128)
    got = w8_linear_tokens(x.to(DEV), codes.to(DEV), scale.to(DEV), group_size=128)
    assert tuple(got.shape) == (tokens, n)
    assert rel_err(got, ref) < PER_KERNEL_REL_TOL


def test_grouped_experts_sorted_pairs():
    from lemoq.kernels.batched_w8 import w8_experts_tokens

    experts, hidden, ffn = 5, 512, 512
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(experts, 2 * ffn, hidden, generator=g) * 0.05
    dn = torch.randn(experts, hidden, ffn, generator=g) * 0.05
    gu_c, gu_s = ops.rtn_quantize_w8(gu, 128)
    dn_c, dn_s = ops.rtn_quantize_w8(dn, 128)
    q = ops.QuantExperts(gu_c, gu_s, dn_c, dn_s, 128)
    # expert 2 has no pair; expert 3 has more pairs than a warp carries through one pass over its rows (16), and an odd count
    ids = torch.tensor([0, 0, 0, 1] + [3] * 37 + [4], dtype=torch.int64)
    x = torch.randn(ids.numel(), hidden, generator=g).half()
    got = w8_experts_tokens(x.to(DEV), ids.to(DEV), gu_c.to(DEV), gu_s.to(DEV), dn_c.to(DEV), dn_s.to(DEV), group_size=128)
    one = torch.ones(1, dtype=torch.float16)
    ref = torch.stack([ops.grouped_moe_w8(x[i], q, ids[i:i + 1], one)[0] for i in range(ids.numel())])
    assert rel_err(got, ref) < PER_KERNEL_REL_TOL


def test_contract_errors():
    from lemoq.kernels.batched_w8 import quantise_tokens, w8_rows_tokens

    with pytest.raises(ValueError):
        quantise_tokens(torch.zeros(2, 2048, device=DEV))  # not fp16
    planes = quantise_tokens(torch.zeros(2, 2048, dtype=torch.float16, device=DEV))
    codes = torch.zeros(3, 8, 2048, dtype=torch.int8, device=DEV)
    scale = torch.zeros(3, 8, 16, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        w8_rows_tokens(planes, 2, codes, scale, group_size=128)  # several experts without segments
    with pytest.raises(NotImplementedError):
        w8_rows_tokens(planes, 2, codes[0, :, :300].contiguous(), scale[0, :, :2].contiguous(), group_size=128)  # K % 512
