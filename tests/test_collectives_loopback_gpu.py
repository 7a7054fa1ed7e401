# SPDX-License-Identifier: Apache-2.0
"""The peer-memory collective kernels and the fused GEMM + collective kernels on ONE GPU.

`create_loopback_contexts(n, bytes)` emulates n ranks in this process: every rank's symmetric arena is a plain
allocation on the same device, so "a peer's memory" is local memory and the kernels run exactly as they do across
NVLink, one emulated rank after the other (flags that a real peer would set are primed before each launch). Every
result is compared with plain PyTorch fp32 math on the same inputs. The multi-process versions of these tests
(tests/test_distributed_gpu.py) need two GPUs; these need one.
"""
import pytest
import torch

import core_scheduler_b200 as cs

C = cs._C
pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def seeded(seed, *shape, dtype=torch.float32):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g).to(dtype)


def each_rank(ctxs, fn):
    """Runs fn(rank, ctx) for every emulated rank in turn, with that rank's flags primed."""
    for r, ctx in enumerate(ctxs):
        ctx.prime_loopback()
        fn(r, ctx)
    torch.cuda.synchronize()
    for ctx in ctxs:
        ctx.check_status()


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("dtype,n", [(torch.float32, 4 * 1000 + 4), (BF, 8 * 4099), (torch.float32, 1 << 20)])
def test_all_reduce_in_the_arena(ranks, dtype, n):
    ctxs = C.create_loopback_contexts(ranks, 32 << 20)
    bufs = [ctx.empty([n], dtype)[0] for ctx in ctxs]
    for r, b in enumerate(bufs):
        b.copy_(seeded(10 + r, n, dtype=dtype))
    expect = sum(seeded(10 + r, n, dtype=dtype).double() for r in range(ranks))
    each_rank(ctxs, lambda r, ctx: ctx.all_reduce_([bufs[r]], "sum"))
    tol = dict(rtol=2e-2, atol=1.5e-1) if dtype == BF else dict(rtol=1e-6, atol=1e-5)
    for b in bufs:
        assert torch.allclose(b.double(), expect, **tol)
    for b in bufs[1:]:
        assert torch.equal(b, bufs[0])  # every rank holds the same bits


@pytest.mark.parametrize("ranks", [2, 8])
def test_all_gather_reduce_scatter_all_to_all(ranks):
    n = 8 * 1031
    ctxs = C.create_loopback_contexts(ranks, 32 << 20)
    for dtype in (torch.float32, BF):
        tol = dict(rtol=2e-2, atol=1.5e-1) if dtype == BF else dict(rtol=1e-6, atol=1e-5)
        # all-gather into one arena block per rank (the owners push their shards)
        dst = [ctx.empty([ranks, n], dtype)[0] for ctx in ctxs]
        each_rank(ctxs, lambda r, ctx: ctx.all_gather_([dst[r][p] for p in range(ranks)], seeded(20 + r, n, dtype=dtype)))
        for d in dst:
            for p in range(ranks):
                assert torch.equal(d[p], seeded(20 + p, n, dtype=dtype))
        # all-gather into ordinary tensors (pull from the peers' staging blocks): staging is written first by everyone
        outs = [[torch.zeros(n, device="cuda", dtype=dtype) for _ in range(ranks)] for _ in range(ranks)]
        src = [ctx.empty([n], dtype)[0] for ctx in ctxs]
        for r in range(ranks):
            src[r].copy_(seeded(30 + r, n, dtype=dtype))
        each_rank(ctxs, lambda r, ctx: ctx.all_gather_(outs[r], src[r]))
        for r in range(ranks):
            for p in range(ranks):
                assert torch.equal(outs[r][p], seeded(30 + p, n, dtype=dtype))
        # reduce-scatter from arena blocks
        send = [ctx.empty([ranks, n], dtype)[0] for ctx in ctxs]
        for r in range(ranks):
            send[r].copy_(seeded(40 + r, ranks, n, dtype=dtype))
        recv = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(ranks)]
        each_rank(ctxs, lambda r, ctx: ctx.reduce_scatter_(recv[r], [send[r][p] for p in range(ranks)], "sum"))
        for r in range(ranks):
            e = sum(seeded(40 + p, ranks, n, dtype=dtype)[r].double() for p in range(ranks))
            assert torch.allclose(recv[r].double(), e, **tol)
        # all-to-all with strided column blocks (pack and unpack inside the transfer)
        rows, cols = 64, 32
        a2a_src = [ctx.empty([rows, cols * ranks], dtype)[0] for ctx in ctxs]
        for r in range(ranks):
            a2a_src[r].copy_(seeded(50 + r, rows, cols * ranks, dtype=dtype))
        a2a_dst = [torch.zeros(rows, cols * ranks, device="cuda", dtype=dtype) for _ in range(ranks)]
        each_rank(ctxs, lambda r, ctx: ctx.all_to_all_([a2a_dst[r][:, p * cols:(p + 1) * cols] for p in range(ranks)],
                                                       [a2a_src[r][:, p * cols:(p + 1) * cols] for p in range(ranks)]))
        for r in range(ranks):
            for p in range(ranks):
                assert torch.equal(a2a_dst[r][:, p * cols:(p + 1) * cols], seeded(50 + p, rows, cols * ranks, dtype=dtype)[:, r * cols:(r + 1) * cols])


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_large_copies_through_the_bulk_engine(ranks):
    """Messages of half a megabyte and more are moved by the cp.async.bulk ring instead of vector loads and stores:
    sizes that are not multiples of the 32 KB stage, rows shorter and longer than a stage."""
    n = 300_008  # 1.2 MB of fp32, 36 full stages and a tail
    ctxs = C.create_loopback_contexts(ranks, 96 << 20)
    launches = C.kernel_launch_count()
    dst = [ctx.empty([ranks, n], torch.float32)[0] for ctx in ctxs]
    each_rank(ctxs, lambda r, ctx: ctx.all_gather_([dst[r][p] for p in range(ranks)], seeded(200 + r, n)))
    for d in dst:
        for p in range(ranks):
            assert torch.equal(d[p], seeded(200 + p, n))
    outs = [[torch.zeros(n, device="cuda") for _ in range(ranks)] for _ in range(ranks)]
    src = [ctx.empty([n], torch.float32)[0] for ctx in ctxs]
    for r in range(ranks):
        src[r].copy_(seeded(210 + r, n))
    each_rank(ctxs, lambda r, ctx: ctx.all_gather_(outs[r], src[r]))
    for r in range(ranks):
        for p in range(ranks):
            assert torch.equal(outs[r][p], seeded(210 + p, n))
    for rows, cols in ((160, 1056), (20, 10_004)):  # 4224-byte rows; 40016-byte rows (one stage and a tail each)
        a2a_src = [ctx.empty([rows, cols * ranks], torch.float32)[0] for ctx in ctxs]
        for r in range(ranks):
            a2a_src[r].copy_(seeded(220 + r, rows, cols * ranks))
        a2a_dst = [torch.zeros(rows, cols * ranks, device="cuda") for _ in range(ranks)]
        each_rank(ctxs, lambda r, ctx: ctx.all_to_all_([a2a_dst[r][:, p * cols:(p + 1) * cols] for p in range(ranks)],
                                                       [a2a_src[r][:, p * cols:(p + 1) * cols] for p in range(ranks)]))
        for r in range(ranks):
            for p in range(ranks):
                assert torch.equal(a2a_dst[r][:, p * cols:(p + 1) * cols], seeded(220 + p, rows, cols * ranks)[:, r * cols:(r + 1) * cols])
    assert C.kernel_launch_count() > launches


@pytest.mark.parametrize("ranks", [2, 4])
def test_reduce_scatter_adamw_all_gather_in_one_kernel(ranks):
    """Arena ranges that start and end inside ownership blocks; block j belongs to rank j % ranks."""
    block = 1024
    n = ranks * block * 3 + 512  # the last block is partial
    ctxs = C.create_loopback_contexts(ranks, 16 << 20)
    grads = [ctx.empty([n], torch.float32)[0] for ctx in ctxs]
    lps = [ctx.empty([n], BF)[0] for ctx in ctxs]
    for r in range(ranks):
        grads[r].copy_(seeded(60 + r, n))
        lps[r].zero_()
    w0 = seeded(70, n)
    blocks = (n + block - 1) // block
    per = (blocks + ranks - 1) // ranks
    padded = torch.zeros(blocks * block, device="cuda")
    padded[:n] = w0
    masters = [torch.zeros(per * block, device="cuda") for _ in range(ranks)]
    for j in range(blocks):
        masters[j % ranks][(j // ranks) * block:(j // ranks + 1) * block] = padded[j * block:(j + 1) * block]
    ms = [torch.zeros(per * block, device="cuda") for _ in range(ranks)]
    vs = [torch.zeros(per * block, device="cuda") for _ in range(ranks)]
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    ranges = [(0, 1280), (1280, 2 * block * ranks + 256), (2 * block * ranks + 256, n)]  # three "buckets"
    for lo, hi in ranges:
        each_rank(ctxs, lambda r, ctx: ctx.sharded_adamw_(grads[r], lps[r], masters[r], ms[r], vs[r], lo, hi, block, lr, b1, b2, eps, wd, 1,
                                                          1.0 / ranks))
    g = sum(seeded(60 + r, n).double() for r in range(ranks)) / ranks
    w = w0.double() * (1 - lr * wd)
    m = (1 - b1) * g
    v = (1 - b2) * g * g
    w = w - lr * (m / (1 - b1)) / ((v / (1 - b2)).sqrt() + eps)
    got = torch.zeros(blocks * block, device="cuda", dtype=torch.float64)
    for j in range(blocks):
        got[j * block:(j + 1) * block] = masters[j % ranks][(j // ranks) * block:(j // ranks + 1) * block].double()
    assert torch.allclose(got[:n], w, rtol=1e-5, atol=1e-6)
    for lp in lps:  # every rank's bf16 working copy received every block
        assert torch.allclose(lp.double(), w, rtol=1e-2, atol=1e-2)


# the last two cases move half a megabyte per chunk: the gather then runs on the bulk engine
@pytest.mark.parametrize("ranks,rows,chunks", [(2, 512, 2), (4, 256, 1), (8, 1024, 4), (2, 2048, 2), (4, 4096, 4)])
@pytest.mark.parametrize("weight_is_rhs", [False, True])
def test_gather_beside_gemm(ranks, rows, chunks, weight_is_rhs):
    """all-gather -> GEMM: rows arrive in chunks announced by flags; the GEMM's loads wait for them."""
    k, n = 256, 384
    ctxs = C.create_loopback_contexts(ranks, 64 << 20)
    fulls = [ctx.empty([ranks * rows, k], BF)[0] for ctx in ctxs]
    shards = [seeded(80 + r, rows, k).mul_(0.5).to(BF) for r in range(ranks)]
    signals = [None] * ranks

    def gather(r, ctx):
        signals[r] = ctx.gather_rows_chunked(shards[r], fulls[r], chunks)

    each_rank(ctxs, gather)
    x = torch.cat(shards).float()
    for f in fulls:
        assert torch.equal(f.float(), x)
    w = seeded(90, k, n).mul_(0.1).to(BF) if weight_is_rhs else seeded(90, n, k).mul_(0.1).to(BF)
    expect = x @ (w.float() if weight_is_rhs else w.float().t())
    ys = [None] * ranks

    def gemm(r, ctx):
        ys[r] = ctx.gemm_on_gathered_chunks(fulls[r], w, weight_is_rhs, 0, None, signals[r])[0]

    each_rank(ctxs, gemm)
    for y in ys:
        assert torch.allclose(y.float(), expect, rtol=2e-2, atol=2e-2)
    assert C.gemm_status()[0] == 0


@pytest.mark.parametrize("ranks,rows", [(2, 256), (4, 512), (8, 256)])
def test_gemm_with_scatter_epilogue_and_slot_sum(ranks, rows):
    """GEMM -> reduce-scatter: bf16 tiles stored into the owners' per-source slots, then summed by the owner."""
    k, n = 192, 256
    m = ranks * rows
    ctxs = C.create_loopback_contexts(ranks, 64 << 20)
    slots = [ctx.empty([ranks, rows, n], BF)[0] for ctx in ctxs]
    xs = [seeded(100 + r, m, k).mul_(0.5).to(BF) for r in range(ranks)]
    ws = [seeded(110 + r, n, k).mul_(0.1).to(BF) for r in range(ranks)]
    residuals = [seeded(120 + r, rows, n).to(BF) for r in range(ranks)]
    each_rank(ctxs, lambda r, ctx: ctx.gemm_scatter_to_slots(xs[r], ws[r], False, slots[r]))
    outs = [None] * ranks

    def total(r, ctx):
        outs[r] = ctx.sum_slots(slots[r], residuals[r])

    each_rank(ctxs, total)
    partial = sum((xs[p].float() @ ws[p].float().t()).to(BF).float() for p in range(ranks))  # bf16 partials, fp32 sum
    for r in range(ranks):
        expect = partial[r * rows:(r + 1) * rows] + residuals[r].float()
        assert torch.allclose(outs[r].float(), expect, rtol=2e-2, atol=6e-2), (outs[r].float() - expect).abs().max().item()
    assert C.gemm_status()[0] == 0
