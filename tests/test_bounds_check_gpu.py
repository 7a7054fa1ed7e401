# SPDX-License-Identifier: Apache-2.0
"""Diagnostic kernel build (-DCS_BOUNDS_CHECK): out-of-range indices are recorded and skipped.

Runs in a child process because the checked library is chosen at import time (CS_BOUNDS_CHECK=1).
The child refuses to launch anything unless the checked kernels are really the ones loaded, so an
out-of-range index can never reach an unchecked kernel.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent(
    """
    import torch
    import core_scheduler_b200 as cs
    C = cs._C
    assert C.bounds_check_enabled(), "checked kernels not loaded"
    s = cs.DynamicScheduler(0, device="cuda")
    T = cs.from_torch
    BF = torch.bfloat16

    # 1. healthy launches leave the report empty (LayerNorm, GELU, embedding, classifier + cross-entropy, attention)
    x = torch.randn(300, 768, device="cuda").to(BF)
    ln = C.layer_norm_init(s, [768])
    with cs.autocast(s, BF):
        y = C.layer_norm_forward(s, ln, T(x))
    C.layer_norm_backward(s, ln, T(x))
    g = C.gelu_init(s)
    C.gelu_forward(s, g, T(x))
    te, pe = C.embedding_init(s, 100, 64), C.embedding_init(s, 16, 64)
    idx = torch.randint(0, 100, (2, 16), device="cuda")
    with cs.autocast(s, BF):
        C.embedding_forward_token_position(s, te, pe, T(idx))
    lin = C.linear_init(s, 128, 512, bias=False)
    ce = C.linear_cross_entropy_init(s, lin, valid_classes=500)
    xs = torch.randn(256, 128, device="cuda").to(BF)
    tg = torch.randint(0, 500, (256,), device="cuda")
    with cs.autocast(s, BF):
        C.linear_cross_entropy_forward(s, ce, T(xs), T(tg))
    C.linear_cross_entropy_backward(s, ce)
    qkv = torch.randn(1, 128, 3 * 2 * 64, device="cuda").to(BF)
    rc, out, lse = C.attention_forward_tcgen05(qkv, 2, 0.125)
    C.attention_backward_tcgen05(qkv, out, torch.randn_like(out), lse, 2, 0.125)
    s.synchronize()
    assert C.bounds_report(True)[0] == 0, C.bounds_report(False)

    # 2. a token id beyond the vocabulary: recorded with kernel id, index and limit; the kernel clamps the read
    bad = idx.clone()
    bad[1, 3] = 100000
    with cs.autocast(s, BF):
        C.embedding_forward_token_position(s, te, pe, T(bad))
    s.synchronize()
    code, kid, block, thread, index, limit = C.bounds_report(True)
    assert (code, kid, index, limit) == (1, 13, 100000, 100), (code, kid, index, limit)

    # 3. a class label beyond the logits row: recorded, the row is skipped, the loss stays finite
    tg2 = tg.clone()
    tg2[5] = 9999
    with cs.autocast(s, BF):
        loss = C.linear_cross_entropy_forward(s, ce, T(xs), T(tg2))
    C.linear_cross_entropy_backward(s, ce)
    s.synchronize()
    code, kid, block, thread, index, limit = C.bounds_report(True)
    assert code == 1 and kid == 15 and index == 9999, (code, kid, index, limit)
    assert torch.isfinite(loss.raw()).all()
    assert C.bounds_report(False)[0] == 0  # the report was cleared
    print("OK bounds")
    """
)


def test_checked_build_records_and_skips_out_of_range_indices():
    lib = os.path.join(ROOT, "core_scheduler_b200", "lib_checked", "libcs_b200.so")
    if not os.path.exists(lib):
        pytest.skip("diagnostic library not built (python -m core_scheduler_b200.build checked)")
    env = dict(os.environ, CS_BOUNDS_CHECK="1", CS_NO_AUTOBUILD="1", PYTHONPATH=ROOT)
    proc = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "OK bounds" in proc.stdout, (proc.stdout + proc.stderr)[-3000:]
