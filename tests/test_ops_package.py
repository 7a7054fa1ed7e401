# SPDX-License-Identifier: Apache-2.0
"""core_scheduler_b200.ops: the object layer over the native ops, checked against PyTorch autograd on the CPU."""
import torch
import torch.nn.functional as F

import core_scheduler_b200 as cs
from core_scheduler_b200 import ops
from helpers import T, attention_reference


def test_block_of_ops_matches_autograd(cpu_scheduler):
    """embedding -> LayerNorm -> Linear -> GeluLinear -> cross-entropy, with every gradient compared."""
    s = cpu_scheduler
    torch.manual_seed(0)
    dtype = torch.float64
    emb = ops.Embedding(s, 50, 16, dtype=dtype)
    ln = ops.LayerNorm(s, 16, dtype=dtype)
    fc1 = ops.Linear(s, 16, 32, bias=True, dtype=dtype)
    fc2 = ops.GeluLinear(s, 32, 50, bias=False, dtype=dtype)
    loss_fn = ops.CrossEntropy(s)
    ids = torch.randint(0, 50, (4, 8))
    target = torch.randint(0, 50, (32,))

    params = {k: v.raw().clone().requires_grad_(True) for k, v in
              dict(emb=emb.weight, g=ln.weight, b=ln.bias, w1=fc1.weight, b1=fc1.bias, w2=fc2.weight).items()}
    x = F.embedding(ids, params["emb"])
    h = F.layer_norm(x, (16,), params["g"], params["b"])
    h = F.linear(h, params["w1"], params["b1"])
    logits = F.linear(F.gelu(h), params["w2"]).view(32, 50)
    expected = F.cross_entropy(logits, target)
    expected.backward()

    y = fc2.forward(fc1.forward(ln.forward(emb.forward(T(ids)))))
    loss = loss_fn.forward(cs._C.utils_view(s, y, [32, 50]), T(target))
    assert torch.allclose(loss.raw(), expected.detach())
    d = cs._C.utils_view(s, loss_fn.backward(), [4, 8, 50])
    d = ln.backward(fc1.backward(fc2.backward(d)))
    emb.backward(d)
    got = dict(emb=emb.grad_weight, g=ln.grad_weight, b=ln.grad_bias, w1=fc1.grad_weight, b1=fc1.grad_bias, w2=fc2.grad_weight)
    for k, g in got.items():
        assert torch.allclose(g.raw(), params[k].grad, atol=1e-10), k
    fc1.zero_grad()
    assert not fc1.grad_weight.defined()


def test_attention_gelu_adamw_and_clipping(cpu_scheduler):
    s = cpu_scheduler
    torch.manual_seed(1)
    q, k, v = (torch.randn(2, 5, 3, 8, dtype=torch.float64) for _ in range(3))
    attn = ops.Attention(s, is_causal=True)
    out = attn.forward(T(q), T(k), T(v))
    assert torch.allclose(out.raw(), attention_reference(q, k, v, causal=True))
    assert [g.raw().shape for g in attn.backward(T(torch.randn_like(q)))] == [q.shape] * 3

    act = ops.GeLU(s)
    x = torch.randn(3, 7, dtype=torch.float64, requires_grad=True)
    F.gelu(x).backward(torch.ones(3, 7, dtype=torch.float64))
    act.forward(T(x.detach()))
    assert torch.allclose(act.backward(T(torch.ones(3, 7, dtype=torch.float64))).raw(), x.grad)

    w = T(torch.ones(16))
    opt = ops.AdamW(s, w, lr=0.1, weight_decay=0.0)
    opt.step(w, T(torch.full((16,), 2.0)))
    assert torch.allclose(w.raw(), torch.full((16,), 0.9), atol=1e-6)  # first step moves by lr along the gradient's sign

    grads = [T(torch.full((4,), 3.0)), T(torch.full((9,), 4.0))]
    norm = ops.clip_grad_norm_(s, grads, max_norm=1.0)
    expected = (4 * 9.0 + 9 * 16.0) ** 0.5
    assert abs(norm.raw().item() - expected) < 1e-5
    assert torch.allclose(grads[0].raw(), torch.full((4,), 3.0 / expected), atol=1e-5)
