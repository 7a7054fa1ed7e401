# SPDX-License-Identifier: Apache-2.0
"""sm_100a kernels against plain PyTorch fp32 references of the same op (GPU only)."""
import math

import pytest
import torch
import torch.nn.functional as F

import core_scheduler_b200 as cs
from helpers import T, TorchGPT2, attention_reference

C = cs._C
pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def bf16_close(a, b, atol=2e-2, rtol=2e-2):
    return torch.allclose(a.float(), b.float(), atol=atol, rtol=rtol)


def test_native_kernels_are_the_path_that_runs(gpu_scheduler):
    s = gpu_scheduler
    before = C.kernel_launch_count()
    st = C.gelu_init(s)
    C.gelu_forward(s, st, T(torch.randn(1024, device="cuda", dtype=BF)))
    s.synchronize()
    assert C.get_backend() == "fused"
    assert C.kernel_launch_count() > before


@pytest.mark.parametrize("rows,d", [(64, 768), (1000, 1024), (37, 1280), (8, 256), (5, 2048), (3, 4096)])
def test_layernorm_forward_backward(gpu_scheduler, rows, d):
    s = gpu_scheduler
    torch.manual_seed(0)
    st = C.layer_norm_init(s, [d])  # fp32 parameters
    st.weight.raw().uniform_(0.5, 1.5)
    st.bias.raw().uniform_(-0.5, 0.5)
    x = torch.randn(rows, d, device="cuda").mul_(2).add_(0.5).to(BF)
    dy = torch.randn(rows, d, device="cuda").to(BF)
    res = torch.randn(rows, d, device="cuda").to(BF)
    xr = x.float().requires_grad_(True)
    w = st.weight.raw().clone().requires_grad_(True)
    b = st.bias.raw().clone().requires_grad_(True)
    yr = F.layer_norm(xr, (d,), w, b)
    yr.backward(dy.float())
    with cs.autocast(s, BF):
        y = C.layer_norm_forward(s, st, T(x))
    dx = C.layer_norm_backward(s, st, T(dy), T(res))
    s.synchronize()
    assert y.raw().dtype == BF
    assert bf16_close(y.raw(), yr)
    assert bf16_close(dx.raw(), xr.grad + res.float(), atol=4e-2)
    assert torch.allclose(st.grad_weight.raw(), w.grad, atol=2e-2 * math.sqrt(rows), rtol=2e-2)
    assert torch.allclose(st.grad_bias.raw(), b.grad, atol=2e-2 * math.sqrt(rows), rtol=2e-2)
    # second micro-step accumulates
    with cs.autocast(s, BF):
        C.layer_norm_forward(s, st, T(x))
    C.layer_norm_backward(s, st, T(dy))
    s.synchronize()
    assert torch.allclose(st.grad_bias.raw(), 2 * b.grad, atol=4e-2 * math.sqrt(rows), rtol=2e-2)


@pytest.mark.parametrize("n", [8, 1000, 1 << 20, (1 << 20) + 3])
def test_gelu_and_add(gpu_scheduler, n):
    s = gpu_scheduler
    x = torch.randn(n, device="cuda").mul_(3).to(BF)
    dy = torch.randn(n, device="cuda").to(BF)
    st = C.gelu_init(s)
    y = C.gelu_forward(s, st, T(x))
    dx = C.gelu_backward(s, st, T(dy))
    xr = x.float().requires_grad_(True)
    yr = F.gelu(xr)
    yr.backward(dy.float())
    s.synchronize()
    assert bf16_close(y.raw(), yr)
    assert bf16_close(dx.raw(), xr.grad)
    if n % 8 == 0:
        z = C.utils_add(s, T(x), T(dy))
        s.synchronize()
        assert bf16_close(z.raw(), x.float() + dy.float())


def test_embedding_token_position(gpu_scheduler):
    s = gpu_scheduler
    V, P, d, B, Tn = 1000, 64, 256, 4, 48
    te, pe = C.embedding_init(s, V, d), C.embedding_init(s, P, d)
    idx = torch.randint(0, V, (B, Tn), device="cuda")
    idx[0, :8] = 7  # duplicates exercise the atomics
    with cs.autocast(s, BF):
        y = C.embedding_forward_token_position(s, te, pe, T(idx))
    ref = te.weight.raw()[idx] + pe.weight.raw()[:Tn][None]
    dy = torch.randn(B, Tn, d, device="cuda").to(BF)
    C.embedding_backward_token_position(s, te, pe, T(dy))
    s.synchronize()
    assert bf16_close(y.raw(), ref)
    gte = torch.zeros(V, d, device="cuda").index_add_(0, idx.reshape(-1), dy.float().reshape(-1, d))
    gpe = torch.zeros(P, d, device="cuda")
    gpe[:Tn] = dy.float().sum(0)
    assert torch.allclose(te.grad_weight.raw(), gte, atol=1e-3)
    assert torch.allclose(pe.grad_weight.raw(), gpe, atol=1e-3)


@pytest.mark.parametrize("n", [1000, 1 << 20])
@pytest.mark.parametrize("amsgrad", [False, True])
def test_adamw_kernel_fp32_master_with_bf16_copy(gpu_scheduler, n, amsgrad):
    from test_optimizer_module import adamw_reference

    s = gpu_scheduler
    w0 = torch.randn(n, device="cuda")
    w = T(w0.clone())
    C.working_copy(s, w, BF)  # creates the bf16 working copy the kernel refreshes
    st = C.adamw_init(s, w, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1, amsgrad=amsgrad)
    wr, m, v = w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)
    vmax = torch.zeros_like(w0) if amsgrad else None
    for t in range(1, 4):
        g = torch.randn(n, device="cuda")
        C.adamw_step(s, st, w, T(g))
        wr, m, v, vmax = adamw_reference(wr, g, m, v, t, 1e-2, 0.9, 0.95, 1e-8, 0.1, vmax)
    s.synchronize()
    assert torch.allclose(w.raw(), wr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(st.m.raw(), m, rtol=1e-4, atol=1e-6)
    assert torch.equal(w.lp(), w.raw().to(BF))


def test_adamw_kernel_bf16_gradients(gpu_scheduler):
    s = gpu_scheduler
    w = T(torch.randn(4096, device="cuda"))
    ref = w.raw().clone()
    st = C.adamw_init(s, w, lr=1e-2, weight_decay=0.0)
    g = torch.randn(4096, device="cuda").to(BF)
    C.adamw_step(s, st, w, T(g))
    s.synchronize()
    # first step of Adam moves every weight by ~lr * sign(g)
    assert torch.allclose(w.raw(), ref - 1e-2 * torch.sign(g.float()), atol=1e-4)


def test_clip_grad_norm_kernels(gpu_scheduler):
    s = gpu_scheduler
    g1 = torch.randn(100000, device="cuda") * 3
    g2 = (torch.randn(5000, device="cuda") * 3).to(BF)
    ref = torch.cat([g1, g2.float()]).norm()
    norm = C.utils_clip_grad_norm_(s, [T(g1), T(g2)], 1.0)
    s.synchronize()
    assert torch.allclose(norm.raw(), ref, rtol=1e-3)
    assert abs(torch.cat([g1, g2.float()]).norm().item() - 1.0) < 2e-2


def test_transposed_working_copy(gpu_scheduler):
    s = gpu_scheduler
    w = T(torch.randn(300, 200, device="cuda"))
    wt = C.working_copy_transposed(s, w, BF)
    s.synchronize()
    assert torch.equal(wt.raw(), w.raw().t().to(BF))


@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (300, 768, 2304), (1024, 3072, 768), (128, 64, 100)])
def test_linear_paths_bf16(gpu_scheduler, M, K, N):
    """Forward (+residual, +GELU companion), dgrad and fp32-accumulated wgrad against fp32 math."""
    s = gpu_scheduler
    torch.manual_seed(1)
    st = C.linear_init(s, K, N, bias=False, gelu_epilogue=True)
    st.weight.raw().normal_(0, 0.05)
    x = torch.randn(M, K, device="cuda").to(BF)
    res = torch.randn(M, N, device="cuda").to(BF)
    dy = torch.randn(M, N, device="cuda").mul_(0.1).to(BF)
    w = st.weight.raw().to(BF).float()
    with cs.autocast(s, BF):
        y = C.linear_forward(s, st, T(x))
    dx = C.linear_backward_input(s, st, T(dy))
    C.linear_backward_parameter(s, st, T(dy))
    with cs.autocast(s, BF):
        C.linear_forward(s, st, T(x))
    C.linear_backward_parameter(s, st, T(dy))  # accumulates
    s.synchronize()
    ref = x.float() @ w.t()
    assert bf16_close(y.raw(), ref, atol=3e-2)
    assert bf16_close(y.companion(), F.gelu(ref), atol=3e-2)
    assert bf16_close(dx.raw(), dy.float() @ w, atol=3e-2)
    gw = dy.float().t() @ x.float()
    assert st.grad_weight.raw().dtype == torch.float32
    assert torch.allclose(st.grad_weight.raw(), 2 * gw, atol=5e-2, rtol=2e-2)
    st2 = C.linear_init(s, K, N, bias=False)
    st2.weight.raw().copy_(st.weight.raw())
    with cs.autocast(s, BF):
        y2 = C.linear_forward(s, st2, T(x), T(res))
    s.synchronize()
    assert bf16_close(y2.raw(), ref + res.float(), atol=4e-2)


def test_gelu_linear_bf16(gpu_scheduler):
    s = gpu_scheduler
    M, K, N = 512, 1024, 256
    st = C.gelu_linear_init(s, K, N, bias=False)
    st.weight.raw().normal_(0, 0.05)
    x = torch.randn(M, K, device="cuda").to(BF)
    dy = torch.randn(M, N, device="cuda").mul_(0.1).to(BF)
    with cs.autocast(s, BF):
        y = C.gelu_linear_forward(s, st, T(x))
    dx = C.gelu_linear_backward_input(s, st, T(dy))
    C.gelu_linear_backward_parameter(s, st, T(dy))
    s.synchronize()
    xr = x.float().requires_grad_(True)
    w = st.weight.raw().to(BF).float().requires_grad_(True)
    yr = F.gelu(xr) @ w.t()
    yr.backward(dy.float())
    assert bf16_close(y.raw(), yr, atol=3e-2)
    assert bf16_close(dx.raw(), xr.grad, atol=3e-2)
    assert torch.allclose(st.grad_weight.raw(), w.grad, atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("rows,d,V,valid", [(256, 128, 512, 500), (1000, 768, 2048, 2048), (130, 256, 1280, 1279)])
def test_fused_classifier_cross_entropy(gpu_scheduler, rows, d, V, valid):
    s = gpu_scheduler
    torch.manual_seed(2)
    lin = C.linear_init(s, d, V, bias=False)
    lin.weight.raw().normal_(0, 0.05)
    st = C.linear_cross_entropy_init(s, lin, valid_classes=valid)
    x = torch.randn(rows, d, device="cuda").to(BF)
    t = torch.randint(0, valid, (rows,), device="cuda")
    t[3] = -100
    with cs.autocast(s, BF):
        loss = C.linear_cross_entropy_forward(s, st, T(x), T(t))
    dx = C.linear_cross_entropy_backward(s, st)
    s.synchronize()
    xr = x.float().requires_grad_(True)
    w = lin.weight.raw().to(BF).float().requires_grad_(True)
    lr = F.cross_entropy((xr @ w.t())[:, :valid], t)
    lr.backward()
    assert abs(loss.raw().item() - lr.item()) < 2e-2
    assert bf16_close(dx.raw(), xr.grad, atol=2e-3, rtol=5e-2)
    assert torch.allclose(lin.grad_weight.raw(), w.grad, atol=2e-3, rtol=5e-2)


def test_attention_bf16_packed(gpu_scheduler):
    s = gpu_scheduler
    B, Tn, H, D = 2, 256, 4, 64
    qkv = torch.randn(B, Tn, 3 * H * D, device="cuda").to(BF)
    st = C.attention_init(s, is_causal=True)
    out = C.attention_forward_packed(s, st, T(qkv), H)
    do = torch.randn(B, Tn, H * D, device="cuda").to(BF)
    dqkv = C.attention_backward_packed(s, st, T(do))
    s.synchronize()
    qr = qkv.float().requires_grad_(True)
    q, k, v = qr.view(B, Tn, 3, H, D).unbind(2)
    ref = attention_reference(q, k, v).reshape(B, Tn, H * D)
    ref.backward(do.float())
    assert bf16_close(out.raw(), ref, atol=3e-2)
    assert bf16_close(dqkv.raw(), qr.grad, atol=5e-2, rtol=5e-2)


def _train_losses(s, backend, steps=4):
    C.set_backend(backend)
    try:
        cs.manual_seed(0)
        cfg = cs.GPT2Config(n_layer=2, n_head=4, n_embd=256, block_size=128, vocab_size=1000, padded_vocab_size=1024)
        m = cs.GPT2(s, cfg)
        flat = C.flatten_parameters(s, m, lp_dtype=BF)
        opt = cs.AdamW(s, m, lr=1e-3, beta1=0.9, beta2=0.95, weight_decay=0.1, flat=flat)
        g = torch.Generator(device="cuda").manual_seed(3)
        ids = torch.randint(0, 1000, (4, 129), device="cuda", generator=g)
        x, y = T(ids[:, :-1].contiguous()), T(ids[:, 1:].contiguous())
        first = {k: v.raw().clone() for k, v in m.named_parameters().items()}
        losses = []
        for _ in range(steps):
            with cs.autocast(s, BF):
                loss = m.forward_loss(s, x, y)
            m.backward_loss(s)
            if not losses:
                s.synchronize()
                grads = {k: v.raw().clone() for k, v in m.named_gradients().items()}
            opt.step(s)
            opt.zero_grad(s)
            losses.append(cs.to_torch(s, loss).item())
        return losses, first, grads, (ids[:, :-1], ids[:, 1:])
    finally:
        C.set_backend("fused")


def test_gpt2_bf16_training_matches_fp32_autograd_and_library_backend(gpu_scheduler):
    s = gpu_scheduler
    fused, params, grads, (ids, lab) = _train_losses(s, "fused")
    lib, _, _, _ = _train_losses(s, "library")
    ref = TorchGPT2(2, 4, 256, 128, 1024, 1000).cuda()
    ref.load_from(params)
    lr = ref(ids, lab)
    lr.backward()
    assert abs(fused[0] - lr.item()) < 3e-2
    assert abs(lib[0] - lr.item()) < 3e-2
    assert fused[-1] < fused[0]
    for a, b in zip(fused, lib):
        assert abs(a - b) < 5e-2
    for k in ("lm_head.weight", "1.mlp.fc2.weight", "0.attn.c_attn.weight", "0.ln1.weight", "wpe.weight"):
        g, r = grads[k].float(), ref.p(k).grad
        err = (g - r).norm() / (r.norm() + 1e-12)
        assert err < 5e-2, (k, err.item())
