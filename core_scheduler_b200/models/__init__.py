# SPDX-License-Identifier: Apache-2.0
"""Model presets. The model itself (`GPT2`) is implemented in C++ (csrc/src/models_gpt2.cpp)."""
from __future__ import annotations

import torch

from .. import _C

PRESETS = {
    # name: (n_layer, n_head, n_embd, block_size, vocab, padded_vocab)
    "tiny": (2, 4, 128, 64, 512, 512),
    "124M": (12, 12, 768, 1024, 50257, 50304),
    "350M": (24, 16, 1024, 1024, 50257, 50304),
    "774M": (36, 20, 1280, 1024, 50257, 50304),
}


def gpt2_config(name: str = "124M", dtype: torch.dtype = torch.float32, fused_classifier: bool = True,
                init_std: float = 0.02) -> "_C.GPT2Config":
    """GPT-2 configuration as the reference's examples build it: untied lm_head, no Linear bias."""
    n_layer, n_head, n_embd, block, vocab, padded = PRESETS[name]
    return _C.GPT2Config(n_layer=n_layer, n_head=n_head, n_embd=n_embd, block_size=block, vocab_size=vocab,
                         padded_vocab_size=padded, use_bias=False, dtype=dtype, init_std=init_std,
                         fused_classifier=fused_classifier)
