# SPDX-License-Identifier: Apache-2.0
"""tcgen05 GEMM kernel: every layout/epilogue against fp32 PyTorch math, including ragged tiles."""
import pytest
import torch
import torch.nn.functional as F

import core_scheduler_b200 as cs

C = cs._C
pytestmark = pytest.mark.gpu
BF = torch.bfloat16
TN, NT = 0, 1
STORE, RESIDUAL, GELU_DUAL, DGELU, STORE_F32, ACCUM_F32, CE = range(7)


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def operands(M, N, K):
    torch.manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, device="cuda").to(BF)
    b = torch.randn(N, K, device="cuda").mul_(0.1).to(BF)
    return a, b


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 768), (300, 2304, 768), (1000, 776, 200), (77, 8, 72),
                                   (4096, 768, 3072), (129, 264, 1032)])
def test_tn_store_and_bias(M, N, K):
    a, b = operands(M, N, K)
    ref = a.float() @ b.float().t()
    d = torch.full((M, N), float("nan"), device="cuda", dtype=BF)
    assert C.gemm_bf16(a, b, d, TN, STORE) == 0
    assert rel(d, ref) < 4e-3
    bias = torch.randn(N, device="cuda").to(BF)
    assert C.gemm_bf16(a, b, d, TN, STORE, bias=bias) == 0
    assert rel(d, ref + bias.float()) < 4e-3
    assert C.gemm_status()[0] == 0


def test_output_padding_is_untouched():
    """Rows/columns outside [M, N] of a strided output must never be written."""
    M, N, K = 200, 520, 128
    a, b = operands(M, N, K)
    big = torch.full((M + 8, N + 16), 7.0, device="cuda", dtype=BF)
    d = big[:M, :N]
    assert C.gemm_bf16(a, b, d, TN, STORE) == 0
    torch.cuda.synchronize()
    assert rel(d, a.float() @ b.float().t()) < 4e-3
    assert (big[M:] == 7).all() and (big[:, N:] == 7).all()


@pytest.mark.parametrize("M,N,K", [(256, 768, 768), (1000, 776, 264)])
def test_tn_residual_gelu_dual_dgelu(M, N, K):
    a, b = operands(M, N, K)
    ref = a.float() @ b.float().t()
    aux = torch.randn(M, N, device="cuda").to(BF)
    d = torch.empty(M, N, device="cuda", dtype=BF)
    assert C.gemm_bf16(a, b, d, TN, RESIDUAL, aux=aux) == 0
    assert rel(d, ref + aux.float()) < 4e-3
    d2 = torch.empty_like(d)
    assert C.gemm_bf16(a, b, d, TN, GELU_DUAL, d2=d2) == 0
    assert rel(d, ref) < 4e-3
    assert rel(d2, F.gelu(d.float())) < 4e-3  # GELU of the stored (rounded) pre-activation
    assert C.gemm_bf16(a, b, d, TN, DGELU, aux=aux) == 0
    x = aux.float().requires_grad_(True)
    F.gelu(x).backward(torch.ones_like(x))
    assert rel(d, ref * x.grad) < 5e-3


@pytest.mark.parametrize("Kr,M,N", [(64, 128, 256), (4096, 768, 2304), (1000, 200, 776), (16384, 768, 768), (520, 1032, 264)])
def test_nt_weight_gradient_store_and_accumulate(Kr, M, N):
    torch.manual_seed(Kr + M + N)
    a = torch.randn(Kr, M, device="cuda").to(BF)
    b = torch.randn(Kr, N, device="cuda").mul_(0.1).to(BF)
    ref = a.float().t() @ b.float()
    d = torch.full((M, N), float("nan"), device="cuda")
    assert C.gemm_bf16(a, b, d, NT, STORE_F32) == 0
    assert rel(d, ref) < 1e-4
    assert C.gemm_bf16(a, b, d, NT, ACCUM_F32) == 0
    assert rel(d, 2 * ref) < 1e-4
    assert C.gemm_status()[0] == 0


def test_tn_fp32_output():
    a, b = operands(256, 512, 4096)
    d = torch.zeros(256, 512, device="cuda")
    assert C.gemm_bf16(a, b, d, TN, STORE_F32) == 0
    assert rel(d, a.float() @ b.float().t()) < 1e-4


@pytest.mark.parametrize("M,V,K,valid", [(256, 1024, 128, 1000), (300, 1288, 256, 1288), (128, 50304, 64, 50257)])
def test_cross_entropy_epilogue_partials(M, V, K, valid):
    a, b = operands(M, V, K)
    tiles = C.gemm_ce_stat_tiles(V)
    stats = torch.full((M, tiles, 2), float("nan"), device="cuda")
    d = torch.empty(M, V, device="cuda", dtype=BF)
    assert C.gemm_bf16(a, b, d, TN, CE, stats=stats, n_valid=valid) == 0
    torch.cuda.synchronize()
    logits = d.float()[:, :valid]
    m = stats[..., 0].max(dim=1).values
    lse = m + torch.log((stats[..., 1] * torch.exp(stats[..., 0] - m[:, None]).nan_to_num(0.0)).sum(1))
    assert torch.allclose(lse, torch.logsumexp(logits, dim=1), atol=2e-3)
    assert rel(d, a.float() @ b.float().t()) < 4e-3


def test_unsupported_shapes_are_declined():
    a = torch.randn(64, 60, device="cuda").to(BF)  # K not a multiple of 8
    b = torch.randn(64, 60, device="cuda").to(BF)
    d = torch.empty(64, 64, device="cuda", dtype=BF)
    assert C.gemm_bf16(a, b, d, TN, STORE) == -1


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (4096, 768, 2304), (1000, 776, 264), (16384, 3072, 768), (100, 264, 136)])
def test_tm_input_gradient_layout(M, N, K):
    """A [M,K] row-major times B [K,N] row-major (the weight as stored): dX = dY * W."""
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(BF)
    b = torch.randn(K, N, device="cuda").mul_(0.1).to(BF)
    d = torch.full((M, N), float("nan"), device="cuda", dtype=BF)
    assert C.gemm_bf16(a, b, d, 2, STORE) == 0
    ref = a.float() @ b.float()
    assert rel(d, ref) < 4e-3
    aux = torch.randn(M, N, device="cuda").to(BF)
    assert C.gemm_bf16(a, b, d, 2, DGELU, aux=aux) == 0
    x = aux.float().requires_grad_(True)
    F.gelu(x).backward(torch.ones_like(x))
    assert rel(d, ref * x.grad) < 5e-3
    assert C.gemm_status()[0] == 0
