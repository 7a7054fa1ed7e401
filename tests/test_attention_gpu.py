# SPDX-License-Identifier: Apache-2.0
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


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 256, 3), (1, 1024, 2), (1, 384, 2)])
def test_backward_matches_reference(B, T, H):
    """dQ, dK, dV written into the packed layout equal autograd through fp32 masked-softmax attention."""
    D = 64
    torch.manual_seed(7 * B + T + H)
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(B, T, H * D, device="cuda").to(BF)
    scale = 1.0 / math.sqrt(D)
    rc, out, lse = C.attention_forward_tcgen05(qkv, H, scale)
    assert rc == 0
    dqkv, delta = C.attention_backward_tcgen05(qkv, out, dout, lse, H, scale)
    torch.cuda.synchronize()
    assert C.attention_status()[0] == 0
    qr = qkv.float().requires_grad_(True)
    q, k, v = qr.view(B, T, 3, H, D).unbind(2)
    ref = attention_reference(q, k, v).reshape(B, T, H * D)
    ref.backward(dout.float())
    ref_delta = (ref.detach() * dout.float()).view(B, T, H, D).sum(-1).permute(0, 2, 1)
    assert torch.allclose(delta, ref_delta, atol=5e-2, rtol=2e-2)
    got, want = dqkv.float().view(B, T, 3, H, D), qr.grad.view(B, T, 3, H, D)
    for i, name in enumerate(("dq", "dk", "dv")):
        err = (got[:, :, i] - want[:, :, i]).abs().max().item()
        ref_mag = want[:, :, i].abs().max().item()
        assert err <= 3e-2 * max(1.0, ref_mag), (name, err, ref_mag)


def test_backward_through_the_op_uses_own_kernels(gpu_scheduler, monkeypatch):
    """With the tcgen05 engine selected, forward_packed/backward_packed run this library's kernels end to end."""
    monkeypatch.setenv("CS_ATTENTION_ENGINE", "tcgen05")
    s = gpu_scheduler
    B, T, H, D = 2, 256, 4, 64
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(BF)
    do = torch.randn(B, T, H * D, device="cuda").to(BF)
    st = C.attention_init(s, is_causal=True)
    before = C.kernel_launch_count()
    out = C.attention_forward_packed(s, st, cs.from_torch(qkv), H)
    dqkv = C.attention_backward_packed(s, st, cs.from_torch(do))
    s.synchronize()
    assert C.kernel_launch_count() - before == 4  # 1 forward + 3 backward launches, no library kernel
    qr = qkv.float().requires_grad_(True)
    q, k, v = qr.view(B, T, 3, H, D).unbind(2)
    ref = attention_reference(q, k, v).reshape(B, T, H * D)
    ref.backward(do.float())
    assert torch.allclose(out.raw().float(), ref, atol=2e-2, rtol=2e-2)
    assert (dqkv.raw().float() - qr.grad).abs().max().item() < 5e-2


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 256, 3), (1, 512, 2)])
def test_non_causal_forward_and_backward_match_reference(B, T, H):
    """The same kernels without the mask: every query attends to every key."""
    D = 64
    torch.manual_seed(11 * B + T + H)
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(B, T, H * D, device="cuda").to(BF)
    scale = 1.0 / math.sqrt(D)
    rc, out, lse = C.attention_forward_tcgen05(qkv, H, scale, causal=False)
    assert rc == 0
    dqkv, _ = C.attention_backward_tcgen05(qkv, out, dout, lse, H, scale, causal=False)
    torch.cuda.synchronize()
    assert C.attention_status()[0] == 0
    qr = qkv.float().requires_grad_(True)
    q, k, v = qr.view(B, T, 3, H, D).unbind(2)
    ref = attention_reference(q, k, v, causal=False).reshape(B, T, H * D)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    s = torch.einsum("bthd,bshd->bhts", q, k) * scale
    assert torch.allclose(lse, torch.logsumexp(s, dim=-1), atol=2e-2, rtol=1e-3)
    got, want = dqkv.float().view(B, T, 3, H, D), qr.grad.view(B, T, 3, H, D)
    for i, name in enumerate(("dq", "dk", "dv")):
        err = (got[:, :, i] - want[:, :, i]).abs().max().item()
        assert err <= 3e-2 * max(1.0, want[:, :, i].abs().max().item()), (name, err)


def test_non_causal_attention_through_the_op_stays_on_own_kernels(gpu_scheduler):
    s = gpu_scheduler
    B, T, H, D = 2, 256, 2, 64
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(BF)
    st = C.attention_init(s, is_causal=False)
    fallbacks = C.library_fallbacks()
    before = C.kernel_launch_count()
    out = C.attention_forward_packed(s, st, cs.from_torch(qkv), H)
    s.synchronize()
    assert C.kernel_launch_count() - before == 1 and C.library_fallbacks() == fallbacks
    q, k, v = qkv.float().view(B, T, 3, H, D).unbind(2)
    assert torch.allclose(out.raw().float(), attention_reference(q, k, v, causal=False).reshape(B, T, H * D), atol=2e-2, rtol=2e-2)
