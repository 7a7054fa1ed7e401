# SPDX-License-Identifier: Apache-2.0
"""Plain PyTorch references used as oracles by the tests."""
import math

import torch
import torch.nn.functional as F


def T(x):
    import core_scheduler_b200 as cs

    return cs.from_torch(x)


def attention_reference(q, k, v, causal=True, scale=None):
    """q,k,v: [B,T,H,D] -> [B,T,H,D], fp32 math with an explicit mask."""
    up = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf, kf, vf = (t.to(up).transpose(1, 2) for t in (q, k, v))
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        Tq, Tk = s.shape[-2:]
        mask = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).transpose(1, 2)


class TorchGPT2(torch.nn.Module):
    """Autograd GPT-2 with the same structure/keys as core_scheduler_b200.GPT2."""

    def __init__(self, n_layer, n_head, n_embd, block_size, padded_vocab, vocab):
        super().__init__()
        self.cfg = (n_layer, n_head, n_embd, block_size, padded_vocab, vocab)
        d = n_embd
        P = {}
        P["wte.weight"] = torch.nn.Parameter(torch.zeros(padded_vocab, d))
        P["wpe.weight"] = torch.nn.Parameter(torch.zeros(block_size, d))
        for l in range(n_layer):
            P[f"{l}.ln1.weight"] = torch.nn.Parameter(torch.ones(d))
            P[f"{l}.ln1.bias"] = torch.nn.Parameter(torch.zeros(d))
            P[f"{l}.attn.c_attn.weight"] = torch.nn.Parameter(torch.zeros(3 * d, d))
            P[f"{l}.attn.c_proj.weight"] = torch.nn.Parameter(torch.zeros(d, d))
            P[f"{l}.ln2.weight"] = torch.nn.Parameter(torch.ones(d))
            P[f"{l}.ln2.bias"] = torch.nn.Parameter(torch.zeros(d))
            P[f"{l}.mlp.fc1.weight"] = torch.nn.Parameter(torch.zeros(4 * d, d))
            P[f"{l}.mlp.fc2.weight"] = torch.nn.Parameter(torch.zeros(d, 4 * d))
        P["lnf.weight"] = torch.nn.Parameter(torch.ones(d))
        P["lnf.bias"] = torch.nn.Parameter(torch.zeros(d))
        P["lm_head.weight"] = torch.nn.Parameter(torch.zeros(padded_vocab, d))
        self.P = torch.nn.ParameterDict({k.replace(".", "/"): v for k, v in P.items()})

    def p(self, key):
        return self.P[key.replace(".", "/")]

    def load_from(self, named):
        with torch.no_grad():
            for k, v in named.items():
                self.p(k).copy_(v.to(self.p(k).dtype))

    def forward(self, ids, labels):
        n_layer, n_head, d, _, padded_vocab, vocab = self.cfg
        B, Tn = ids.shape
        x = self.p("wte.weight")[ids] + self.p("wpe.weight")[:Tn][None]
        for l in range(n_layer):
            a = F.layer_norm(x, (d,), self.p(f"{l}.ln1.weight"), self.p(f"{l}.ln1.bias"))
            qkv = a @ self.p(f"{l}.attn.c_attn.weight").t()
            q, k, v = qkv.view(B, Tn, 3, n_head, d // n_head).unbind(2)
            ctx = attention_reference(q, k, v).reshape(B, Tn, d).to(x.dtype)
            x = x + ctx @ self.p(f"{l}.attn.c_proj.weight").t()
            b = F.layer_norm(x, (d,), self.p(f"{l}.ln2.weight"), self.p(f"{l}.ln2.bias"))
            h = F.gelu(b @ self.p(f"{l}.mlp.fc1.weight").t())
            x = x + h @ self.p(f"{l}.mlp.fc2.weight").t()
        x = F.layer_norm(x, (d,), self.p("lnf.weight"), self.p("lnf.bias"))
        logits = x @ self.p("lm_head.weight").t()
        logits = logits[..., :vocab]
        up = torch.float64 if logits.dtype == torch.float64 else torch.float32
        return F.cross_entropy(logits.reshape(B * Tn, -1).to(up), labels.reshape(-1))
