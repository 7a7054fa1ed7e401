# SPDX-License-Identifier: Apache-2.0
"""Op numerics on the CPU (ATen path) against PyTorch autograd, mirroring the reference's unit tests."""
import math

import pytest
import torch
import torch.nn.functional as F

import core_scheduler_b200 as cs
from helpers import T, attention_reference

C = cs._C


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_matches_autograd(cpu_scheduler, dtype, bias):
    s = cpu_scheduler
    torch.manual_seed(1)
    st = C.linear_init(s, 4, 16, bias=bias, dtype=dtype)
    x = torch.randn(32, 3, 4, dtype=dtype, requires_grad=True)
    w = st.weight.raw().clone().requires_grad_(True)
    b = st.bias.raw().clone().requires_grad_(True) if bias else None
    y = C.linear_forward(s, st, T(x.detach()))
    yr = F.linear(x, w, b)
    dy = torch.randn_like(yr)
    yr.backward(dy)
    dx = C.linear_backward_input(s, st, T(dy))
    C.linear_backward_parameter(s, st, T(dy))
    assert torch.allclose(y.raw(), yr)
    assert torch.allclose(dx.raw(), x.grad)
    assert torch.allclose(st.grad_weight.raw(), w.grad)
    if bias:
        assert torch.allclose(st.grad_bias.raw(), b.grad)


def test_linear_gradient_accumulates_then_clears(cpu_scheduler):
    s = cpu_scheduler
    st = C.linear_init(s, 8, 8, bias=False)
    x = torch.randn(5, 8)
    dy = torch.randn(5, 8)
    for _ in range(2):
        C.linear_forward(s, st, T(x))
        C.linear_backward_parameter(s, st, T(dy))
    assert torch.allclose(st.grad_weight.raw(), 2 * dy.t() @ x, atol=1e-5)
    st.zero_grad()
    assert not st.grad_weight.defined()


def test_linear_residual_extension(cpu_scheduler):
    s = cpu_scheduler
    st = C.linear_init(s, 8, 8, bias=False)
    x, r = torch.randn(5, 8), torch.randn(5, 8)
    y = C.linear_forward(s, st, T(x), T(r))
    assert torch.allclose(y.raw(), x @ st.weight.raw().t() + r, atol=1e-6)


@pytest.mark.parametrize("bias", [False, True])
def test_gelu_linear_matches_autograd(cpu_scheduler, bias):
    s = cpu_scheduler
    torch.manual_seed(2)
    st = C.gelu_linear_init(s, 128, 64, bias=bias, dtype=torch.float64)
    x = torch.randn(12, 3, 128, dtype=torch.float64, requires_grad=True)
    w = st.weight.raw().clone().requires_grad_(True)
    b = st.bias.raw().clone().requires_grad_(True) if bias else None
    y = C.gelu_linear_forward(s, st, T(x.detach()))
    yr = F.linear(F.gelu(x), w, b)
    dy = torch.randn_like(yr)
    yr.backward(dy)
    dx = C.gelu_linear_backward_input(s, st, T(dy))
    C.gelu_linear_backward_parameter(s, st, T(dy))
    assert torch.allclose(y.raw(), yr)
    assert torch.allclose(dx.raw(), x.grad)
    assert torch.allclose(st.grad_weight.raw(), w.grad)
    if bias:
        assert torch.allclose(st.grad_bias.raw(), b.grad)


def test_gelu_linear_weight_gradient_accumulates_correctly(cpu_scheduler):
    """The reference's accumulate graph replaces the gradient; two micro-steps must add up here."""
    s = cpu_scheduler
    st = C.gelu_linear_init(s, 16, 8, bias=False, dtype=torch.float64)
    x = torch.randn(4, 16, dtype=torch.float64)
    dy = torch.randn(4, 8, dtype=torch.float64)
    for _ in range(2):
        C.gelu_linear_forward(s, st, T(x))
        C.gelu_linear_backward_input(s, st, T(dy))
        C.gelu_linear_backward_parameter(s, st, T(dy))
    assert torch.allclose(st.grad_weight.raw(), 2 * dy.t() @ F.gelu(x))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_layer_norm_matches_autograd(cpu_scheduler, dtype):
    s = cpu_scheduler
    torch.manual_seed(3)
    st = C.layer_norm_init(s, [384], dtype=dtype)
    st.weight.raw().uniform_(0.5, 1.5)
    st.bias.raw().uniform_(-0.5, 0.5)
    x = torch.randn(16, 24, 384, dtype=dtype, requires_grad=True)
    w = st.weight.raw().clone().requires_grad_(True)
    b = st.bias.raw().clone().requires_grad_(True)
    y = C.layer_norm_forward(s, st, T(x.detach()))
    yr = F.layer_norm(x, (384,), w, b)
    dy = torch.randn_like(yr)
    yr.backward(dy)
    dx = C.layer_norm_backward(s, st, T(dy))
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else {}
    assert torch.allclose(y.raw(), yr, **tol)
    assert torch.allclose(dx.raw(), x.grad, **tol)
    assert torch.allclose(st.grad_weight.raw(), w.grad, atol=1e-4 if dtype == torch.float32 else 1e-10)
    assert torch.allclose(st.grad_bias.raw(), b.grad, atol=1e-4 if dtype == torch.float32 else 1e-10)


def test_layer_norm_backward_with_residual(cpu_scheduler):
    s = cpu_scheduler
    st = C.layer_norm_init(s, [64], dtype=torch.float64)
    x = torch.randn(10, 64, dtype=torch.float64, requires_grad=True)
    C.layer_norm_forward(s, st, T(x.detach()))
    dy, r = torch.randn(10, 64, dtype=torch.float64), torch.randn(10, 64, dtype=torch.float64)
    F.layer_norm(x, (64,), st.weight.raw(), st.bias.raw()).backward(dy)
    dx = C.layer_norm_backward(s, st, T(dy), T(r))
    assert torch.allclose(dx.raw(), x.grad + r)


@pytest.mark.parametrize("n", [128, 512, 1024])
def test_gelu_forward_backward(cpu_scheduler, n):
    s = cpu_scheduler
    st = C.gelu_init(s)
    x = torch.randn(2, n, requires_grad=True)
    y = C.gelu_forward(s, st, T(x.detach()))
    yr = F.gelu(x)
    dy = torch.randn_like(yr)
    yr.backward(dy)
    dx = C.gelu_backward(s, st, T(dy))
    assert torch.allclose(y.raw(), yr)
    assert torch.allclose(dx.raw(), x.grad, atol=1e-6)


def test_embedding_forward_backward(cpu_scheduler):
    s = cpu_scheduler
    st = C.embedding_init(s, 4095, 512)
    idx = torch.randint(0, 3, (2, 1024))
    w = st.weight.raw().clone().requires_grad_(True)
    y = C.embedding_forward(s, st, T(idx))
    yr = F.embedding(idx, w)
    dy = torch.randn_like(yr)
    yr.backward(dy)
    C.embedding_backward(s, st, T(dy))
    assert torch.allclose(y.raw(), yr)
    assert torch.allclose(st.grad_weight.raw(), w.grad, atol=1e-4)


def test_embedding_padding_idx_gets_no_gradient(cpu_scheduler):
    s = cpu_scheduler
    st = C.embedding_init(s, 10, 8, padding_idx=0)
    assert st.weight.raw()[0].abs().sum() == 0
    idx = torch.tensor([[0, 1, 0, 2]])
    C.embedding_forward(s, st, T(idx))
    C.embedding_backward(s, st, T(torch.ones(1, 4, 8)))
    g = st.grad_weight.raw()
    assert g[0].abs().sum() == 0 and g[1].sum() == 8


def test_token_position_embedding(cpu_scheduler):
    s = cpu_scheduler
    te, pe = C.embedding_init(s, 50, 16), C.embedding_init(s, 12, 16)
    idx = torch.randint(0, 50, (3, 7))
    y = C.embedding_forward_token_position(s, te, pe, T(idx))
    assert torch.allclose(y.raw(), te.weight.raw()[idx] + pe.weight.raw()[:7][None])
    dy = torch.randn(3, 7, 16)
    C.embedding_backward_token_position(s, te, pe, T(dy))
    ref = torch.zeros(12, 16)
    ref[:7] = dy.sum(0)
    assert torch.allclose(pe.grad_weight.raw(), ref, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_cross_entropy_matches_torch(cpu_scheduler, dtype):
    s = cpu_scheduler
    st = C.cross_entropy_init(s)
    x = torch.randn(2048, 384, dtype=dtype, requires_grad=True)
    t = torch.randint(0, 384, (2048,))
    t[5] = -100
    loss = C.cross_entropy_forward(s, st, T(x.detach()), T(t))
    lr = F.cross_entropy(x, t)
    lr.backward()
    dx = C.cross_entropy_backward(s, st)
    assert torch.allclose(loss.raw(), lr)
    assert torch.allclose(dx.raw(), x.grad, atol=1e-7)


def test_cross_entropy_under_autocast_uses_fp32_statistics(cpu_scheduler):
    s = cpu_scheduler
    st = C.cross_entropy_init(s)
    x = torch.randn(64, 100).bfloat16()
    t = torch.randint(0, 100, (64,))
    with cs.autocast(s, torch.bfloat16):
        loss = C.cross_entropy_forward(s, st, T(x), T(t))
    assert loss.raw().dtype == torch.float32
    assert torch.allclose(loss.raw(), F.cross_entropy(x.float(), t), atol=1e-5)
    assert C.cross_entropy_backward(s, st).raw().dtype == torch.bfloat16


def test_linear_cross_entropy_matches_composition(cpu_scheduler):
    s = cpu_scheduler
    lin = C.linear_init(s, 32, 96, bias=False, dtype=torch.float64)
    st = C.linear_cross_entropy_init(s, lin, valid_classes=90)
    x = torch.randn(4, 10, 32, dtype=torch.float64, requires_grad=True)
    t = torch.randint(0, 90, (4, 10))
    t[0, 0] = -100
    w = lin.weight.raw().clone().requires_grad_(True)
    loss = C.linear_cross_entropy_forward(s, st, T(x.detach()), T(t))
    lr = F.cross_entropy((x @ w.t())[..., :90].reshape(40, 90), t.reshape(-1))
    lr.backward()
    dx = C.linear_cross_entropy_backward(s, st)
    assert torch.allclose(loss.raw(), lr)
    assert torch.allclose(dx.raw(), x.grad)
    assert torch.allclose(lin.grad_weight.raw(), w.grad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_attention_matches_masked_softmax(cpu_scheduler, dtype):
    s = cpu_scheduler
    B, Tn, H, D = 15, 7, 8, 8
    st = C.attention_init(s, is_causal=True, scale=1 / math.sqrt(D))
    q, k, v = (torch.randn(B, Tn, H, D, dtype=dtype, requires_grad=True) for _ in range(3))
    out = C.attention_forward(s, st, T(q.detach()), T(k.detach()), T(v.detach()))
    ref = attention_reference(q, k, v)
    do = torch.randn_like(ref)
    ref.backward(do)
    dq, dk, dv = C.attention_backward(s, st, T(do))
    tol = dict(atol=1e-5, rtol=1e-4)
    assert torch.allclose(out.raw(), ref.detach(), **tol)
    assert torch.allclose(dq.raw(), q.grad, **tol)
    assert torch.allclose(dk.raw(), k.grad, **tol)
    assert torch.allclose(dv.raw(), v.grad, **tol)


def test_attention_packed_equals_split(cpu_scheduler):
    s = cpu_scheduler
    B, Tn, H, D = 2, 9, 4, 8
    qkv = torch.randn(B, Tn, 3 * H * D, requires_grad=True)
    st = C.attention_init(s, is_causal=True)
    out = C.attention_forward_packed(s, st, T(qkv.detach()), H)
    q, k, v = qkv.view(B, Tn, 3, H, D).unbind(2)
    ref = attention_reference(q, k, v).reshape(B, Tn, H * D)
    do = torch.randn_like(ref)
    ref.backward(do)
    dqkv = C.attention_backward_packed(s, st, T(do))
    assert torch.allclose(out.raw(), ref.detach(), atol=1e-5)
    assert torch.allclose(dqkv.raw(), qkv.grad, atol=1e-5)


def test_utils_cat_sum_clip(cpu_scheduler):
    s = cpu_scheduler
    a, b = torch.randn(8, 8, 8), torch.randn(8, 8, 8)
    assert torch.equal(C.utils_cat(s, [T(a), T(b)], 1).raw(), torch.cat([a, b], 1))
    assert torch.allclose(C.utils_sum(s, T(a), [0, 2]).raw(), a.sum((0, 2)))
    g1, g2 = torch.randn(100) * 10, torch.randn(50) * 10
    r1, r2 = g1.clone(), g2.clone()
    total = torch.nn.utils.clip_grad_norm_([torch.nn.Parameter(r1), torch.nn.Parameter(r2)], 1.0)  # no grads: returns 0
    ref_norm = torch.cat([g1, g2]).norm()
    norm = C.utils_clip_grad_norm_(s, [T(g1), T(g2)], 1.0)
    assert torch.allclose(norm.raw(), ref_norm)
    assert torch.allclose(torch.cat([g1, g2]).norm(), torch.tensor(1.0), atol=1e-4)
    del total


def test_utils_views_and_factories(cpu_scheduler):
    s = cpu_scheduler
    x = torch.arange(24.0).reshape(2, 12)
    parts = C.utils_split(s, T(x), 4, 1)
    assert len(parts) == 3 and torch.equal(parts[1].raw(), x[:, 4:8])
    assert C.utils_view(s, T(x), [4, 6]).raw().shape == (4, 6)
    assert C.utils_broadcast_to(s, T(torch.ones(1, 3)), [5, 3]).raw().shape == (5, 3)
    assert torch.equal(C.utils_arange(s, 0, 5).raw(), torch.arange(5))
    assert C.utils_zeros(s, [2, 2], torch.float32).raw().sum() == 0
    r = C.utils_randint(s, 0, 7, [100]).raw()
    assert r.min() >= 0 and r.max() < 7
    assert torch.allclose(C.utils_add(s, T(x), T(x)).raw(), 2 * x)
    assert torch.allclose(C.utils_linalg_vector_norm(s, T(x), 2.0).raw(), x.norm())


def test_autocast_linear_layernorm_embedding(cpu_scheduler):
    s = cpu_scheduler
    lin = C.linear_init(s, 16, 8, bias=True)  # fp32 parameters
    x = torch.randn(4, 16)
    with cs.autocast(s, torch.bfloat16):
        y = C.linear_forward(s, lin, T(x))
    assert y.raw().dtype == torch.bfloat16
    ref = F.linear(x.bfloat16(), lin.weight.raw().bfloat16(), lin.bias.raw().bfloat16())
    assert torch.allclose(y.raw().float(), ref.float(), atol=2e-2)
    dy = torch.randn(4, 8).bfloat16()
    dx = C.linear_backward_input(s, lin, T(dy))  # outside the guard: uses the stamp
    C.linear_backward_parameter(s, lin, T(dy))
    assert dx.raw().dtype == torch.bfloat16
    assert lin.grad_weight.raw().dtype == torch.float32  # stored in the master dtype
    ln = C.layer_norm_init(s, [16])
    with cs.autocast(s, torch.bfloat16):
        z = C.layer_norm_forward(s, ln, T(x.bfloat16()))
    assert torch.allclose(z.raw().float(), F.layer_norm(x.bfloat16().float(), (16,)), atol=2e-2)
    emb = C.embedding_init(s, 10, 16)
    with cs.autocast(s, torch.bfloat16):
        e = C.embedding_forward(s, emb, T(torch.tensor([[1, 2]])))
    assert e.raw().dtype == torch.bfloat16
