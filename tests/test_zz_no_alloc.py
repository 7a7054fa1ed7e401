# SPDX-License-Identifier: Apache-2.0
"""The allocation-free C entry point, called through its exported symbol.

Some users of the library cannot allocate device memory at the point where they need a kernel:
a host loop that reserved everything at start-up, a plugin inside a process whose allocator it
does not own, a C or ctypes client without torch. For them `cs_layernorm_backward_noalloc`
runs LayerNorm backward with its scratch in a fixed array inside the library. This test calls it
twice in a row through ctypes (raw pointers, no framework objects on the way in) and checks the
results against the regular LayerNorm backward of the framework and against PyTorch's fp32
autograd of the same op, and that the free device memory is the same before and after a call. It is collected last so that a
failure here cannot hide another test's result in a run that stops at the first failure.
"""
import ctypes
import os

import pytest
import torch

import core_scheduler_b200 as cs

C = cs._C
pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _lib():
    path = os.path.join(os.path.dirname(cs.__file__), "lib", "libcs_b200.so")
    lib = ctypes.CDLL(path)
    fn = lib.cs_layernorm_backward_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    return fn


def _case(rows, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, d, device="cuda", generator=g).mul_(1.5).add_(0.25).to(BF)
    dy = torch.randn(rows, d, device="cuda", generator=g).to(BF)
    res = torch.randn(rows, d, device="cuda", generator=g).to(BF)
    gamma = torch.rand(d, device="cuda", generator=g) + 0.5
    return x, dy, res, gamma


def _fp32_autograd(x, dy, res, gamma):
    """dx (+ residual gradient), dgamma, dbeta of LayerNorm from PyTorch's fp32 autograd."""
    xf = x.float().requires_grad_(True)
    g = gamma.clone().requires_grad_(True)
    b = torch.zeros_like(gamma).requires_grad_(True)
    torch.nn.functional.layer_norm(xf, (x.shape[1],), g, b, 1e-5).backward(dy.float())
    return xf.grad + res.float(), g.grad, b.grad


def _framework_backward(s, x, dy, res, gamma):
    st = C.layer_norm_init(s, [x.shape[1]])
    st.weight.raw().copy_(gamma)
    with cs.autocast(s, BF):
        C.layer_norm_forward(s, st, cs.from_torch(x))
    dx = C.layer_norm_backward(s, st, cs.from_torch(dy), cs.from_torch(res))
    s.synchronize()
    return dx.raw(), st.grad_weight.raw(), st.grad_bias.raw()


@pytest.mark.parametrize("rows,d", [(4096, 768), (333, 1280), (16, 2048)])
def test_no_alloc_layernorm_backward_matches_framework_twice(gpu_scheduler, rows, d):
    fn = _lib()
    s = gpu_scheduler
    for call in range(2):  # two calls in a row share the built-in scratch
        x, dy, res, gamma = _case(rows, d, seed=10 * call + 1)
        ref_dx, ref_dg, ref_db = _framework_backward(s, x, dy, res, gamma)
        fp_dx, fp_dg, fp_db = _fp32_autograd(x, dy, res, gamma)
        xf = x.float()
        mean = xf.mean(1).contiguous()
        rstd = torch.rsqrt(xf.var(1, unbiased=False) + 1e-5).contiguous()
        dx = torch.empty_like(x)
        dgamma = torch.full((d,), float("nan"), device="cuda")
        dbeta = torch.full((d,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        if call == 1:  # every one-time set-up happened in the first call: from here on nothing may be allocated
            free_before = torch.cuda.mem_get_info()[0]
        rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), res.data_ptr(),
                dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), 0, rows, d, None)
        assert rc == 0
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == free_before
        # fp32 oracle (bf16 inputs and output: a few bf16 ulps on dx; the column sums grow with sqrt(rows))
        assert torch.allclose(dx.float(), fp_dx, atol=6e-2, rtol=3e-2)
        assert torch.allclose(dgamma, fp_dg, atol=3e-2 * rows ** 0.5, rtol=3e-2)
        assert torch.allclose(dbeta, fp_db, atol=3e-2 * rows ** 0.5, rtol=3e-2)
        assert torch.allclose(dx.float(), ref_dx.float(), atol=4e-2, rtol=2e-2)
        scale = rows ** 0.5
        assert torch.allclose(dgamma, ref_dg, atol=2e-2 * scale, rtol=2e-2)
        assert torch.allclose(dbeta, ref_db, atol=2e-2 * scale, rtol=2e-2)
        # accumulate mode adds to what is there
        rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), None,
                dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), 1, rows, d, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(dbeta, 2 * ref_db, atol=4e-2 * scale, rtol=2e-2)


def test_no_alloc_rejects_sizes_beyond_the_scratch():
    fn = _lib()
    t = torch.zeros(8, device="cuda")
    p = t.data_ptr()
    assert fn(p, p, p, p, p, None, p, p, p, 0, 1, 4096, None) == -1   # wider than the built-in scratch
    assert fn(p, p, p, p, p, None, p, p, p, 0, 1, 100, None) == -1    # not a multiple of 8
    assert fn(None, p, p, p, p, None, p, p, p, 0, 1, 64, None) == -2  # missing pointer
