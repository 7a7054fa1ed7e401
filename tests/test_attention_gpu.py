"""tcgen05 causal attention forward kernel against fp32 masked-softmax attention."""
import math

import pytest
import torch

import core_scheduler_b200 as cs
from helpers import attention_reference

C = cs._C
pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 256, 3), (2, 1024, 4), (1, 384, 2)])
def test_forward_matches_reference(B, T, H):
    D = 64
    torch.manual_seed(B * 1000 + T + H)
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(BF)
    rc, out, lse = C.attention_forward_tcgen05(qkv, H, 1.0 / math.sqrt(D))
    torch.cuda.synchronize()
    assert rc == 0
    assert C.attention_status()[0] == 0
    q, k, v = qkv.float().view(B, T, 3, H, D).unbind(2)
    ref = attention_reference(q, k, v).reshape(B, T, H * D)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    s = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(D)
    mask = torch.ones(T, T, dtype=torch.bool, device="cuda").tril()
    ref_lse = torch.logsumexp(s.masked_fill(~mask, float("-inf")), dim=-1)
    assert torch.allclose(lse, ref_lse, atol=2e-2, rtol=1e-3)


def test_unsupported_shapes_are_declined():
    qkv = torch.randn(1, 100, 3 * 2 * 64, device="cuda").to(BF)  # T not a multiple of 128
    rc, _, _ = C.attention_forward_tcgen05(qkv, 2, 0.125)
    assert rc == -1
    qkv = torch.randn(1, 128, 3 * 2 * 32, device="cuda").to(BF)  # head dimension 32
    rc, _, _ = C.attention_forward_tcgen05(qkv, 2, 0.125)
    assert rc == -1
