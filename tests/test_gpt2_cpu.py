# SPDX-License-Identifier: Apache-2.0
"""End-to-end tiny GPT-2 on the CPU in fp32: loss/gradient parity with an autograd model, one
optimizer step and a save/load round trip (the plumbing configuration)."""
import torch

import core_scheduler_b200 as cs
from helpers import T, TorchGPT2

C = cs._C


def make(s, fused=True, dtype=torch.float32):
    cfg = cs.GPT2Config(n_layer=2, n_head=4, n_embd=128, block_size=64, vocab_size=512, padded_vocab_size=512,
                        dtype=dtype, fused_classifier=fused)
    cs.manual_seed(0)
    return cfg, cs.GPT2(s, cfg)


def test_tiny_gpt2_matches_autograd(cpu_scheduler):
    s = cpu_scheduler
    cfg, m = make(s, dtype=torch.float64)
    ref = TorchGPT2(2, 4, 128, 64, 512, 512).double()
    ref.load_from({k: v.raw() for k, v in m.named_parameters().items()})
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (2, 64), generator=g)
    lab = torch.roll(ids, -1, 1)
    loss = m.forward_loss(s, T(ids), T(lab))
    m.backward_loss(s)
    lr = ref(ids, lab)
    lr.backward()
    assert torch.allclose(loss.raw().double(), lr.detach(), atol=1e-9)
    grads = m.named_gradients()
    for k in m.parameter_names():
        assert torch.allclose(grads[k].raw(), ref.p(k).grad, atol=1e-8), k


def test_unfused_classifier_path_agrees(cpu_scheduler):
    s = cpu_scheduler
    _, a = make(s, fused=True)
    _, b = make(s, fused=False)
    ids = torch.randint(0, 512, (2, 64))
    lab = torch.roll(ids, -1, 1)
    la = a.forward_loss(s, T(ids), T(lab)); a.backward_loss(s)
    lb = b.forward_loss(s, T(ids), T(lab)); b.backward_loss(s)
    assert torch.allclose(la.raw(), lb.raw(), atol=1e-5)
    ga, gb = a.named_gradients(), b.named_gradients()
    for k in a.parameter_names():
        assert torch.allclose(ga[k].raw(), gb[k].raw(), atol=1e-5), k


def test_logits_forward_and_manual_backward(cpu_scheduler):
    s = cpu_scheduler
    _, m = make(s)
    ids = torch.randint(0, 512, (2, 64))
    logits = m.forward(s, T(ids))
    assert logits.raw().shape == (2, 64, 512)
    m.backward(s, T(torch.randn(2 * 64, 512)))
    assert m.named_gradients()["wte.weight"].defined()


def test_training_step_and_checkpoint(cpu_scheduler, tmp_path):
    s = cpu_scheduler
    _, m = make(s)
    opt = cs.AdamW(s, m, lr=1e-3, beta1=0.9, beta2=0.95, weight_decay=0.1)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (2, 64), generator=g)
    lab = torch.roll(ids, -1, 1)
    losses = []
    for _ in range(4):
        loss = m.forward_loss(s, T(ids), T(lab))
        m.backward_loss(s)
        opt.step(s)
        opt.zero_grad(s)
        losses.append(cs.to_torch(s, loss).item())
    assert losses[-1] < losses[0]
    path = str(tmp_path / "gpt2.parquet")
    m.save(path)
    keep = {k: v.raw().clone() for k, v in m.named_parameters().items()}
    for v in m.named_parameters().values():
        v.raw().zero_()
    m.load(path)
    for k, v in m.named_parameters().items():
        assert torch.equal(v.raw(), keep[k]), k


def test_gradient_accumulation_over_micro_steps(cpu_scheduler):
    s = cpu_scheduler
    _, m = make(s)
    ids = torch.randint(0, 512, (2, 64))
    lab = torch.roll(ids, -1, 1)
    m.forward_loss(s, T(ids), T(lab)); m.backward_loss(s)
    once = {k: v.raw().clone() for k, v in m.named_gradients().items()}
    m.forward_loss(s, T(ids), T(lab)); m.backward_loss(s)
    for k, v in m.named_gradients().items():
        assert torch.allclose(v.raw(), 2 * once[k], atol=1e-5), k
