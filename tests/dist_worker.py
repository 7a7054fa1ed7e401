# SPDX-License-Identifier: Apache-2.0
"""Multi-rank test body. Launched by tests/test_distributed*.py through torch.distributed.run:

    python -m torch.distributed.run --standalone ... tests/dist_worker.py <device> <case>

Every case asserts on every rank and prints `OK <case>` from rank 0 when all ranks passed.
"""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import core_scheduler_b200 as cs  # noqa: E402
from core_scheduler_b200.parallel import init_distributed  # noqa: E402

C = cs._C
T = cs.from_torch


def seeded(seed, *shape, dtype=torch.float32, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype).to(device)


def make_comm(device, nvp2p=False, arena_mb=256):
    comm, rank, world, local_rank = init_distributed(device)
    if device == "cuda" and nvp2p:
        pg = dist.distributed_c10d._get_default_group()
        comm = C.comm_from_process_group(pg.group_name, "cuda", True)
        C.create_symmetric_context(comm, arena_mb << 20)
    s = cs.DynamicScheduler(local_rank if device == "cuda" else 0, device=device)
    return comm, rank, world, s


def case_all_reduce(device, nvp2p):
    comm, rank, world, s = make_comm(device, nvp2p)
    for dtype in (torch.float32, torch.bfloat16) if device == "cuda" else (torch.float32, torch.float64):
        # every tensor of a multi-tensor call gets the reduced value, the last one included
        xs = [seeded(100 * rank + i, 128 * (i + 1), dtype=dtype, device=device) for i in range(3)]
        expect = [sum(seeded(100 * r + i, 128 * (i + 1), dtype=dtype, device=device).double() for r in range(world)) for i in range(3)]
        hs = [T(x.clone()) for x in xs]
        C.all_reduce(s, comm, hs, "sum")
        for h, e in zip(hs, expect):
            got = cs.to_torch(s, h).double()
            assert torch.allclose(got, e, rtol=2e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-1 if dtype == torch.bfloat16 else 1e-6), (rank, dtype)
        h = T(xs[0].clone())
        C.all_reduce(s, comm, [h], "avg")
        assert torch.allclose(cs.to_torch(s, h).double(), expect[0] / world, rtol=2e-2, atol=1e-1 if dtype == torch.bfloat16 else 1e-6)
    # large message (8 MiB) on GPUs
    if device == "cuda":
        big = seeded(rank, 1 << 21, device=device)
        e = sum(seeded(r, 1 << 21, device=device) for r in range(world))
        h = T(big.clone())
        C.all_reduce(s, comm, [h], "sum")
        assert torch.allclose(cs.to_torch(s, h), e, atol=1e-4)


def case_all_reduce_arena(device, nvp2p):
    """In-place all-reduce on ranges of the symmetric arena (the data-parallel gradient path), odd sizes included."""
    comm, rank, world, s = make_comm(device, True)
    ctx = C.create_symmetric_context(comm, 64 << 20)
    for dtype, n in ((torch.float32, 4 * 1000 + 4), (torch.float32, 1 << 20), (torch.bfloat16, 8 * 777), (torch.float32, 4 * 12345)):
        buf, off, nb = ctx.empty([n], dtype)
        buf.copy_(seeded(50 * rank + 1, n, dtype=dtype, device=device))
        expect = sum(seeded(50 * r + 1, n, dtype=dtype, device=device).double() for r in range(world))
        torch.cuda.synchronize()
        h = T(buf)
        C.all_reduce(s, comm, [h], "sum")
        s.synchronize()
        tol = dict(rtol=2e-2, atol=1e-1) if dtype == torch.bfloat16 else dict(rtol=1e-6, atol=1e-5)
        assert torch.allclose(buf.double(), expect, **tol), (rank, dtype, n, (buf.double() - expect).abs().max().item())
        C.all_reduce(s, comm, [h], "avg")
        s.synchronize()
        assert torch.allclose(buf.double(), expect, **tol), (rank, "avg", n)  # (sum over identical copies) / world
        ctx.release(off, nb)
    ctx.check_status()


def case_collectives_arena(device, nvp2p):
    """All-gather, reduce-scatter and all-reduce on buffers that live in the symmetric arena (the paths that
    write through the multicast mapping when there is one), each run twice: the kernels reduce in a fixed
    order, so the second run must reproduce the first bit for bit."""
    comm, rank, world, s = make_comm(device, True)
    ctx = C.create_symmetric_context(comm, 96 << 20)
    expect_mc = os.environ.get("CS_EXPECT_MULTICAST")
    if expect_mc is not None:
        assert ctx.has_multicast == (expect_mc == "1"), (ctx.has_multicast, ctx.virtual_memory)
        if expect_mc == "1":
            C.set_multicast_min_ranks(2)  # a pair prefers peer loads by default; this case is about the multimem kernels
    for dtype, n in ((torch.float32, 4 * 3001), (torch.bfloat16, 8 * 4099), (torch.float32, 1 << 20)):
        tol = dict(rtol=2e-2, atol=1e-1) if dtype == torch.bfloat16 else dict(rtol=1e-6, atol=1e-5)
        # all-gather: every rank's shard lands in slot `rank` of one arena block on every rank
        src, so, sb = ctx.empty([n], dtype)
        dst, do, db = ctx.empty([world, n], dtype)
        src.copy_(seeded(7 * rank + 3, n, dtype=dtype, device=device))
        torch.cuda.synchronize()
        results = []
        for _ in range(2):
            dst.zero_()
            torch.cuda.synchronize()
            C.all_gather(s, comm, [[T(dst[p]) for p in range(world)]], [T(src)])
            s.synchronize()
            results.append(dst.clone())
        for p in range(world):
            assert torch.equal(results[0][p], seeded(7 * p + 3, n, dtype=dtype, device=device)), (rank, p, dtype, n)
        assert torch.equal(results[0], results[1])
        # reduce-scatter: chunk p of every rank's arena block is summed into rank p's output
        send, so2, sb2 = ctx.empty([world, n], dtype)
        send.copy_(seeded(11 * rank + 5, world, n, dtype=dtype, device=device))
        torch.cuda.synchronize()
        outs = []
        for _ in range(2):
            out = torch.zeros(n, dtype=dtype, device=device)
            C.reduce_scatter(s, comm, [T(out)], [[T(send[p]) for p in range(world)]], "sum")
            s.synchronize()
            outs.append(out)
        e = sum(seeded(11 * r + 5, world, n, dtype=dtype, device=device)[rank].double() for r in range(world))
        assert torch.allclose(outs[0].double(), e, **tol), (rank, dtype, n)
        assert torch.equal(outs[0], outs[1])
        # all-reduce in place, twice from the same inputs
        buf, bo, bb = ctx.empty([n], dtype)
        sums = []
        for _ in range(2):
            buf.copy_(seeded(13 * rank + 1, n, dtype=dtype, device=device))
            torch.cuda.synchronize()
            C.all_reduce(s, comm, [T(buf)], "sum")
            s.synchronize()
            sums.append(buf.clone())
        e = sum(seeded(13 * r + 1, n, dtype=dtype, device=device).double() for r in range(world))
        assert torch.allclose(sums[0].double(), e, **tol), (rank, dtype, n)
        assert torch.equal(sums[0], sums[1])
        for off, nb in ((so, sb), (do, db), (so2, sb2), (bo, bb)):
            ctx.release(off, nb)
    ctx.check_status()


def case_bucket(device, nvp2p):
    comm, rank, world, s = make_comm(device, nvp2p)
    bucket = cs.AllReduceBucket(1024 * 4, "sum")  # 1024 fp32 elements
    xs = [T(torch.full((400,), float(rank + 1 + i), device=device)) for i in range(5)]
    for x in xs:
        bucket.push_back(s, comm, x)
    assert bucket.launches() == 1  # 3 x 400 elements crossed the threshold once; two tensors still queued
    bucket.sync(s, comm)           # the partial last bucket must be flushed in the same step
    assert bucket.launches() == 2
    total_rank = sum(range(1, world + 1))
    for i, x in enumerate(xs):
        assert torch.allclose(cs.to_torch(s, x), torch.full((400,), float(total_rank + world * i), device=device)), (rank, i)


def case_bucket_arena_order(device, nvp2p):
    """Views of one arena queued in mixed address order are each reduced exactly once."""
    comm, rank, world, s = make_comm(device, nvp2p)
    arena = torch.zeros(4 * 128, device=device)
    views = [arena[i * 128:i * 128 + 100] for i in range(4)]  # 28-element padding after each
    for i, v in enumerate(views):
        v.fill_(float(rank + 1 + i))
    bucket = cs.AllReduceBucket(1 << 30, "sum")
    # descending overall, with one ascending pair (like LayerNorm weight/bias pushed after a matrix)
    for idx in (3, 1, 2, 0):
        bucket.push_back(s, comm, T(views[idx]))
    bucket.sync(s, comm)
    s.synchronize()
    base = sum(range(1, world + 1))
    for i, v in enumerate(views):
        assert torch.allclose(v, torch.full((100,), float(base + world * i), device=device)), (rank, i, v[:3])
    assert bucket.launches() == 1


def case_bucket_gradients_bias(device, nvp2p):
    """Bucketed gradients of a model with biases equal the sum of every rank's local gradients, for several
    bucket thresholds. A bias is pushed right after its weight, so a bucket often closes between the two; a merge
    of arena views that bridged the gap would then reduce the bias in this bucket and again in the next."""
    comm, rank, world, s = make_comm(device, nvp2p)
    g = torch.Generator().manual_seed(23)
    ids = torch.randint(0, 128, (world, 2, 33), generator=g).to(device)

    def build():
        cs.manual_seed(3)
        cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=128, padded_vocab_size=128, use_bias=True)
        m = cs.GPT2(s, cfg)
        symmetric = symm and device == "cuda" and nvp2p
        return m, (C.flatten_symmetric(s, m, comm) if symmetric else C.flatten_parameters(s, m))

    symm = False
    ref, rflat = build()
    symm = True
    for r in range(world):  # the sum over ranks, accumulated locally
        ref.forward_loss(s, T(ids[r][:, :-1].contiguous()), T(ids[r][:, 1:].contiguous()))
        ref.backward_loss(s)
    s.synchronize()
    expect = {k: v.raw().double().clone() for k, v in ref.named_gradients().items()}
    assert any(k.endswith(".bias") for k in expect)
    for threshold in (1, 20 << 10, 48 << 10, 64 << 10, 100 << 10, 200 << 10, 1 << 30):
        model, flat = build()
        bucket = cs.AllReduceBucket(threshold, "sum")
        sync = cs.GradientSync(comm, bucket, True)
        model.forward_loss(s, T(ids[rank][:, :-1].contiguous()), T(ids[rank][:, 1:].contiguous()))
        model.backward_loss(s, sync)
        bucket.sync(s, comm)
        s.synchronize()
        for k, v in model.named_gradients().items():
            got = v.raw().double()
            err = (got - expect[k]).abs().max().item()
            rel = 1e-4 if device == "cpu" else 5e-3
            assert err <= 1e-5 + rel * expect[k].abs().max().item(), (rank, threshold, k, err)


def case_all_gather(device, nvp2p):
    comm, rank, world, s = make_comm(device, nvp2p)
    send = T(seeded(rank + 1, 128, device=device))
    recv = [T(torch.zeros(128, device=device)) for _ in range(world)]
    C.all_gather(s, comm, [recv], [send])
    for r in range(world):
        assert torch.allclose(cs.to_torch(s, recv[r]), seeded(r + 1, 128, device=device)), (rank, r)


def case_reduce_scatter(device, nvp2p):
    comm, rank, world, s = make_comm(device, nvp2p)
    send = [T(seeded(10 * rank + p, 128, device=device)) for p in range(world)]
    recv = T(torch.zeros(128, device=device))
    C.reduce_scatter(s, comm, [recv], [send], "sum")
    expect = sum(seeded(10 * r + rank, 128, device=device) for r in range(world))
    assert torch.allclose(cs.to_torch(s, recv), expect, atol=1e-5), rank


def case_all_to_all(device, nvp2p):
    comm, rank, world, s = make_comm(device, nvp2p)
    send = [T(seeded(10 * rank + p, 128, device=device)) for p in range(world)]
    recv = [T(torch.zeros(128, device=device)) for _ in range(world)]
    C.all_to_all(s, comm, recv, send)
    for p in range(world):
        assert torch.allclose(cs.to_torch(s, recv[p]), seeded(10 * p + rank, 128, device=device)), (rank, p)
    if device == "cuda" and nvp2p:
        # pack/unpack fused: strided [rows, cols] column blocks of one symmetric buffer go straight
        # into strided column blocks of the destination
        ctx_rows, cols = 64, 32
        symm = comm_symmetric_tensor(comm, [ctx_rows, cols * world], torch.float32)
        symm.copy_(seeded(500 + rank, ctx_rows, cols * world, device=device))
        dst = torch.zeros(ctx_rows, cols * world, device=device)
        send2 = [T(symm[:, p * cols:(p + 1) * cols]) for p in range(world)]
        recv2 = [T(dst[:, p * cols:(p + 1) * cols]) for p in range(world)]
        C.all_to_all(s, comm, recv2, send2)
        s.synchronize()
        for p in range(world):
            src = seeded(500 + p, ctx_rows, cols * world, device=device)[:, rank * cols:(rank + 1) * cols]
            assert torch.allclose(dst[:, p * cols:(p + 1) * cols], src), (rank, p)


_symm_keep = []


def comm_symmetric_tensor(comm, sizes, dtype):
    ctx = C.create_symmetric_context(comm, 64 << 20)
    t, off, nbytes = ctx.empty(sizes, dtype)
    _symm_keep.append(ctx)
    return t


def assert_same_training(model, ref, init, rank, amp):
    """Parameters after a few optimizer steps agree.

    On the CPU (fp32, deterministic) the comparison is elementwise. On GPUs bf16 rounding plus
    atomics whose order varies (attention backward, embedding and split-K accumulation) make
    individual elements flip by one bf16 ulp, which Adam's normalised update can turn into a
    different sign for near-zero gradients; there the check is on the update as a whole: its
    relative error and the share of elements that moved differently."""
    pa, pb = model.named_parameters(), ref.named_parameters()
    for k in pa:
        a, b = pa[k].raw().float(), pb[k].raw().float()
        if not amp:
            assert torch.allclose(a, b, atol=1e-5), (rank, k, (a - b).abs().max().item())
            continue
        upd = (b - init[k]).norm().item() + 1e-12
        err = (a - b).norm().item() / upd
        frac = ((a - b).abs() > 2e-3).float().mean().item()
        assert err < 0.25 and frac < 0.02, (rank, k, err, frac)


def tiny_model(s, seed=0):
    cs.manual_seed(seed)
    cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=128, padded_vocab_size=128)
    return cfg, cs.GPT2(s, cfg)


def case_dp_training(device, nvp2p):
    """Two-rank data-parallel steps equal single-process steps on the concatenated batch."""
    comm, rank, world, s = make_comm(device, nvp2p)
    _, model = tiny_model(s)
    _, ref = tiny_model(s)
    amp = device == "cuda"
    if amp:
        flat = C.flatten_symmetric(s, model, comm) if nvp2p else C.flatten_parameters(s, model, lp_dtype=torch.bfloat16)
        rflat = C.flatten_parameters(s, ref, lp_dtype=torch.bfloat16)
    else:
        flat, rflat = C.flatten_parameters(s, model), C.flatten_parameters(s, ref)
    opt = cs.AdamW(s, model, lr=1e-2, weight_decay=0.1, flat=flat)
    ropt = cs.AdamW(s, ref, lr=1e-2, weight_decay=0.1, flat=rflat)
    opt.set_grad_scale(1.0 / world)
    ropt.set_grad_scale(1.0 / world)
    bucket = cs.AllReduceBucket(64 * 1024, "sum")
    sync = cs.GradientSync(comm, bucket, True)
    s.synchronize()
    init = {k: v.raw().float().clone() for k, v in ref.named_parameters().items()}
    g = torch.Generator().manual_seed(7)
    for step in range(3):
        ids = torch.randint(0, 128, (world, 2, 33), generator=g).to(device)
        mine = ids[rank]
        def run(m, x):
            if amp:
                with cs.autocast(s, torch.bfloat16):
                    return m.forward_loss(s, T(x[:, :-1].contiguous()), T(x[:, 1:].contiguous()))
            return m.forward_loss(s, T(x[:, :-1].contiguous()), T(x[:, 1:].contiguous()))
        run(model, mine)
        model.backward_loss(s, sync)
        bucket.sync(s, comm)
        opt.step(s)
        opt.zero_grad(s)
        for r in range(world):  # reference: accumulate every rank's micro-batch locally
            run(ref, ids[r])
            ref.backward_loss(s)
        ropt.step(s)
        ropt.zero_grad(s)
    s.synchronize()
    assert_same_training(model, ref, init, rank, amp)
    assert bucket.launches() >= 3


def case_trainer(device, nvp2p):
    """parallel.GPT2Trainer: two data-parallel ranks follow one process that accumulates both micro-batches; the
    tensor-parallel trainer's loss falls on every rank."""
    from core_scheduler_b200.parallel import GPT2Trainer

    comm, rank, world, s = make_comm(device, nvp2p)
    cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=128, padded_vocab_size=128)
    kind = "nvp2p" if nvp2p else "nccl"
    dp = GPT2Trainer(cfg, comm, world, int(os.environ.get("LOCAL_RANK", "0")), mode="dp", collectives=kind, device=device, lr=1e-2,
                     bucket_mb=0.0625, scheduler=s)
    alone = GPT2Trainer(cfg, None, 1, 0, mode="dp", device=device, lr=1e-2, scheduler=s)
    alone.optimizer.set_grad_scale(1.0 / world)
    init = {k: v.raw().float().clone() for k, v in alone.model.named_parameters().items()}
    g = torch.Generator().manual_seed(13)
    for step in range(3):
        ids = torch.randint(0, 128, (world, 2, 33), generator=g).to(device)
        dp.step(T(ids[rank][:, :-1].contiguous()), T(ids[rank][:, 1:].contiguous()))
        for r in range(world):  # the single process accumulates every rank's micro-batch before its update
            x, y = T(ids[r][:, :-1].contiguous()), T(ids[r][:, 1:].contiguous())
            if alone.amp:
                with cs.autocast(s, torch.bfloat16):
                    alone.model.forward_loss(s, x, y)
            else:
                alone.model.forward_loss(s, x, y)
            alone.model.backward_loss(s)
        alone.optimizer.step(s)
        alone.optimizer.zero_grad(s)
    s.synchronize()
    assert_same_training(dp.model, alone.model, init, rank, dp.amp)
    assert dp.bucket.launches() >= 3

    tp = GPT2Trainer(cfg, comm, world, int(os.environ.get("LOCAL_RANK", "0")), mode="tp", collectives=kind, device=device, lr=1e-2,
                     scheduler=s)
    ids = torch.randint(0, 128, (2 * world, 33), generator=torch.Generator().manual_seed(17)).to(device)
    losses = [tp.step(T(ids[:, :-1].contiguous()), T(ids[:, 1:].contiguous())).raw().float().item() for _ in range(5)]
    assert losses[-1] < losses[0] - 0.2, losses
    # sequence parallel: each rank's loss is the mean over its own share of the token rows


def case_tp_trainer_uneven(device, nvp2p):
    """The tensor-parallel trainer with shards of unequal size (3 heads over 2 ranks). Its parameter and gradient arenas
    sit in symmetric memory ahead of the activation buffers; ranks that allocated different sizes there would address
    each other's buffers at shifted offsets. The loss of a repeated batch starts at ln(vocabulary) and falls."""
    import math

    from core_scheduler_b200.parallel import GPT2Trainer

    comm, rank, world, s = make_comm(device, True)
    cfg = cs.GPT2Config(n_layer=2, n_head=3, n_embd=192, block_size=128, vocab_size=512, padded_vocab_size=512)
    tp = GPT2Trainer(cfg, comm, world, int(os.environ.get("LOCAL_RANK", "0")), mode="tp", collectives="nvp2p", device=device, lr=3e-3,
                     scheduler=s, max_tokens=16 * 128)
    sizes = [torch.zeros(1, dtype=torch.int64, device=device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([tp.flat.total], dtype=torch.int64, device=device))
    assert len({int(t.item()) for t in sizes}) > 1, "the case needs shards of different sizes"
    ids = torch.randint(0, 512, (16, 129), generator=torch.Generator().manual_seed(19)).to(device)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    losses = [tp.step(T(x), T(y)).raw().float().item() for _ in range(8)]
    tp.check_device_status()
    assert all(math.isfinite(v) for v in losses), losses
    assert abs(losses[0] - math.log(512)) < 0.5, losses
    assert losses[-1] < losses[0] - 0.3, losses
    tp.close()


def case_loader_shards_by_rank(device, nvp2p):
    """rows / world rows per rank starting at rank * rows / world, split again over the workers, batches handed out
    worker by worker (the reference's arithmetic, src/data/dataloader.cpp:371-420); iterations per epoch = rows / (batch * world)."""
    import shutil

    import pyarrow as pa
    import pyarrow.parquet as pq

    comm, rank, world, s = make_comm(device, nvp2p)
    directory = f"/tmp/cs_loader_{os.environ.get('MASTER_PORT', '0')}"
    rows_per_file, cols = [10, 6, 16], 8  # 32 rows in three files; boundaries do not coincide with the shards
    if rank == 0:
        os.makedirs(directory, exist_ok=True)
        start = 0
        for i, rows in enumerate(rows_per_file):
            ids = [[(start + r) * 1000 + c for c in range(cols)] for r in range(rows)]
            table = pa.table({"input_ids": pa.array(ids, type=pa.list_(pa.int32())),
                              "labels": pa.array([[v + 1 for v in row] for row in ids], type=pa.list_(pa.int32()))})
            pq.write_table(table, os.path.join(directory, f"data-{i:05d}-of-00003.parquet"))
            start += rows
    dist.barrier()
    ds = C.LlmDataset(directory)
    assert ds.size() == 32
    loader = C.LlmDataLoader(ds, comm, 2, 2, False)  # 16 rows per rank, 8 per worker, 4 batches of 2 per worker
    assert loader.iterations_per_epoch() == 32 // (2 * world)
    base = rank * (32 // world)
    per_worker = (32 // world) // 2
    seen = [(loader.load(s)["input_ids"].raw()[:, 0] // 1000).tolist() for _ in range(8)]
    expected = []
    for i in range(4):
        for w in range(2):
            first = base + w * per_worker + 2 * i
            expected.append([first, first + 1])
    assert seen == expected, (rank, seen, expected)
    del loader
    dist.barrier()
    if rank == 0:
        shutil.rmtree(directory, ignore_errors=True)


def case_resume_smaller_world(device, nvp2p):
    """After a lost rank the job restarts from the last checkpoint with fewer ranks: the checkpoint is rank-agnostic
    (full parameters and moments, written by one rank), so one process that accumulates the micro-batches of both
    former ranks continues exactly where the two-rank job would have."""
    import shutil

    comm, rank, world, s = make_comm(device, nvp2p)
    directory = f"/tmp/cs_resume_{os.environ.get('MASTER_PORT', '0')}"
    g = torch.Generator().manual_seed(11)
    batches = [torch.randint(0, 128, (world, 2, 33), generator=g) for _ in range(3)]

    def micro_step(m, x, sync=None):
        m.forward_loss(s, T(x[:, :-1].contiguous()), T(x[:, 1:].contiguous()))
        m.backward_loss(s, sync) if sync is not None else m.backward_loss(s)

    _, model = tiny_model(s)
    opt = cs.AdamW(s, model, lr=1e-2, weight_decay=0.1, flat=C.flatten_parameters(s, model))
    opt.set_grad_scale(1.0 / world)
    bucket = cs.AllReduceBucket(64 * 1024, "sum")
    sync = cs.GradientSync(comm, bucket, True)

    def dp_step(ids):
        micro_step(model, ids[rank], sync)
        bucket.sync(s, comm)
        opt.step(s)
        opt.zero_grad(s)

    for ids in batches[:2]:
        dp_step(ids)
    meta = C.CheckpointMeta()
    meta.step, meta.data_cursor, meta.world_size, meta.model = 2, 2, world, "tiny"
    C.save_training_state(s, directory, model, opt, meta, rank, 0)  # every rank drains, rank 0 writes
    dist.barrier()
    dp_step(batches[2])  # the uninterrupted two-rank job
    s.synchronize()

    # the restarted job: one rank, a different initialisation, everything from the files
    _, alone = tiny_model(s, seed=99)
    opt1 = cs.AdamW(s, alone, lr=1e-2, weight_decay=0.1, flat=C.flatten_parameters(s, alone))
    got = C.load_training_state(s, directory, alone, opt1)
    assert got.step == 2 and got.world_size == world
    opt1.set_grad_scale(1.0 / got.world_size)  # the global batch stays the same: accumulate the former ranks' micro-batches
    for r in range(got.world_size):
        micro_step(alone, batches[got.data_cursor][r])
    opt1.step(s)
    opt1.zero_grad(s)
    s.synchronize()
    pa, pb = alone.named_parameters(), model.named_parameters()
    for k in pa:
        a, b = pa[k].raw().float(), pb[k].raw().float()
        assert torch.allclose(a, b, atol=1e-5), (rank, k, (a - b).abs().max().item())
    dist.barrier()
    if rank == 0:
        shutil.rmtree(directory, ignore_errors=True)


def case_zero_training(device, nvp2p):
    """ZeRO (fused reduce-scatter + AdamW + all-gather) equals replicated data-parallel AdamW."""
    comm, rank, world, s = make_comm(device, True)
    _, model = tiny_model(s)
    _, ref = tiny_model(s)
    flat = C.flatten_symmetric(s, model, comm)
    rflat = C.flatten_parameters(s, ref, lp_dtype=torch.bfloat16)
    opt = C.ZeroAdamW(s, model, flat, comm, lr=1e-2, weight_decay=0.1)
    ropt = cs.AdamW(s, ref, lr=1e-2, weight_decay=0.1, flat=rflat)
    ropt.set_grad_scale(1.0 / world)
    s.synchronize()
    init = {k: v.raw().float().clone() for k, v in ref.named_parameters().items()}
    g = torch.Generator().manual_seed(11)
    for step in range(3):
        ids = torch.randint(0, 128, (world, 2, 33), generator=g).to(device)
        with cs.autocast(s, torch.bfloat16):
            model.forward_loss(s, T(ids[rank][:, :-1].contiguous()), T(ids[rank][:, 1:].contiguous()))
        model.backward_loss(s)
        opt.step(s)
        opt.zero_grad(s)
        for r in range(world):
            with cs.autocast(s, torch.bfloat16):
                ref.forward_loss(s, T(ids[r][:, :-1].contiguous()), T(ids[r][:, 1:].contiguous()))
            ref.backward_loss(s)
        ropt.step(s)
        ropt.zero_grad(s)
    opt.gather_master(s)
    s.synchronize()
    assert_same_training(model, ref, init, rank, True)
    pa, pb = model.named_parameters(), ref.named_parameters()
    for k in pa:  # the bf16 working copies every rank received match its fp32 masters
        assert torch.allclose(pa[k].lp().float(), pa[k].raw().float(), atol=1e-2, rtol=1e-2), (rank, k)


def case_zero_bucketed(device, nvp2p):
    """The sharded optimizer driven per bucket from the backward pass (reduce-scatter + AdamW + all-gather of every bucket
    beside the remaining backward work) equals replicated data-parallel AdamW; its per-rank shard files merge into the
    per-parameter optimizer table of the replicated optimizer."""
    import shutil

    from core_scheduler_b200.utils.checkpoint import merge_zero, read_parameters

    comm, rank, world, s = make_comm(device, True)
    _, model = tiny_model(s)
    _, ref = tiny_model(s)
    flat = C.flatten_symmetric(s, model, comm)
    rflat = C.flatten_parameters(s, ref, lp_dtype=torch.bfloat16)
    opt = C.ZeroAdamW(s, model, flat, comm, lr=1e-2, weight_decay=0.1)
    bucket = cs.AllReduceBucket(48 * 1024, "sum")
    bucket.attach_sharded_optimizer(opt)
    sync = cs.GradientSync(comm, bucket, True)
    ropt = cs.AdamW(s, ref, lr=1e-2, weight_decay=0.1, flat=rflat)
    ropt.set_grad_scale(1.0 / world)
    s.synchronize()
    init = {k: v.raw().float().clone() for k, v in ref.named_parameters().items()}
    g = torch.Generator().manual_seed(11)
    for step in range(3):
        ids = torch.randint(0, 128, (world, 2, 33), generator=g).to(device)
        with cs.autocast(s, torch.bfloat16):
            model.forward_loss(s, T(ids[rank][:, :-1].contiguous()), T(ids[rank][:, 1:].contiguous()))
        model.backward_loss(s, sync)
        bucket.sync(s, comm)
        opt.step(s)
        opt.zero_grad(s)
        for r in range(world):
            with cs.autocast(s, torch.bfloat16):
                ref.forward_loss(s, T(ids[r][:, :-1].contiguous()), T(ids[r][:, 1:].contiguous()))
            ref.backward_loss(s)
        ropt.step(s)
        ropt.zero_grad(s)
    assert bucket.launches() >= 6  # several buckets per step
    opt.gather_master(s)
    s.synchronize()
    assert_same_training(model, ref, init, rank, True)
    # shard files -> per-parameter table
    directory = f"/tmp/cs_zero_merge_{os.environ.get('MASTER_PORT', '0')}"
    os.makedirs(f"{directory}/zero_rank{rank}", exist_ok=True)
    opt.save(f"{directory}/zero_rank{rank}/optimizer.parquet")
    if rank == 0:
        model.save(f"{directory}/model.parquet")
    dist.barrier()
    merged = merge_zero([read_parameters(f"{directory}/zero_rank{r}/optimizer.parquet") for r in range(world)],
                        read_parameters(f"{directory}/model.parquet"))
    assert merged["__step__"][0] == 3
    rstate = ropt.named_state_tensors()
    for k, p in model.named_parameters().items():
        assert torch.allclose(torch.from_numpy(merged[f"{k}.master"].copy()).to(device), p.raw().float().reshape(-1), atol=1e-6), (rank, k)
        for what in ("m", "v"):
            got = torch.from_numpy(merged[f"{k}.{what}"].copy()).to(device)
            want = rstate[f"{k}.{what}"].raw().float().reshape(-1)
            err = (got - want).norm().item() / (want.norm().item() + 1e-12)
            assert err < 0.2, (rank, k, what, err)
    dist.barrier()
    if rank == 0:
        shutil.rmtree(directory, ignore_errors=True)


def head_range(H, rank, world):
    """Heads of `rank`: the first H % world ranks own one more (same rule as the library)."""
    base, extra = divmod(H, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def tp_slice(name, t, rank, world, cfg):
    """The part of a full GPT-2 parameter (or gradient) that tensor-parallel rank `rank` owns."""
    H, d = cfg.n_head, cfg.n_embd
    D = d // H
    h0, h1 = head_range(H, rank, world)
    if name.endswith("c_attn.weight"):
        return t.view(3, H, D, d)[:, h0:h1].reshape(3 * (h1 - h0) * D, d)
    if name.endswith("c_proj.weight"):
        return t[:, h0 * D:h1 * D]
    if name.endswith("fc1.weight"):
        return t[rank * 4 * d // world:(rank + 1) * 4 * d // world]
    if name.endswith("fc2.weight"):
        return t[:, rank * 4 * d // world:(rank + 1) * 4 * d // world]
    if name == "lm_head.weight" and cfg.padded_vocab_size % (8 * world) == 0:  # vocabulary-parallel classifier
        rows = cfg.padded_vocab_size // world
        return t[rank * rows:(rank + 1) * rows]
    return t


def full_key(k):
    return k.replace(".c_attn", ".attn.c_attn").replace(".c_proj", ".attn.c_proj").replace(".fc1", ".mlp.fc1").replace(".fc2", ".mlp.fc2")


def shard_full_into_tp(full, tp_model, rank, world, cfg):
    """Copies the matching slices of a full GPT-2's parameters into this rank's TP model."""
    fp, tpp = full.named_parameters(), tp_model.named_parameters()
    for k, dst in tpp.items():
        dst.raw().copy_(tp_slice(k, fp[full_key(k)].raw(), rank, world, cfg))


def full_grad_slice(name, g, rank, world, cfg):
    return tp_slice(name, g, rank, world, cfg)


def case_tp_training_fused(device, nvp2p):
    """Same check at a size where the fused all-gather+GEMM / GEMM+reduce-scatter kernels engage."""
    case_tp_training(device, True, batch_per_rank=16, expect_fused=True)


def case_tp_uneven_heads(device, nvp2p):
    """Three heads over two ranks (2 + 1): the split GPT-2 774M needs for 20 heads over 8 ranks."""
    case_tp_training(device, nvp2p, n_head=3, n_embd=96)


def case_tp_uneven_heads_fused(device, nvp2p):
    """Uneven heads (2 + 1, head dimension 64) at a size where the fused GEMM + collective kernels engage."""
    case_tp_training(device, True, batch_per_rank=16, expect_fused=True, n_head=3, n_embd=192)


def case_tp_training(device, nvp2p, batch_per_rank=2, expect_fused=False, n_head=4, n_embd=64):
    """Tensor-parallel GPT-2 (sequence-parallel activations) reproduces the single-device loss and gradients."""
    comm, rank, world, s = make_comm(device, nvp2p)
    amp = device == "cuda"
    dtype = torch.float32 if amp else torch.float64
    cs.manual_seed(3)
    cfg = cs.GPT2Config(n_layer=2, n_head=n_head, n_embd=n_embd, block_size=32, vocab_size=128, padded_vocab_size=128, dtype=dtype)
    full = cs.GPT2(s, cfg)
    tp = C.TPGPT2(s, cfg, comm)
    s.synchronize()
    assert tp.head_range() == (head_range(n_head, rank, world)[0], head_range(n_head, rank, world)[1] - head_range(n_head, rank, world)[0])
    shard_full_into_tp(full, tp, rank, world, cfg)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 128, (batch_per_rank * world, 33), generator=g).to(device)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    bucket = cs.AllReduceBucket(1 << 16, "sum")
    sync = cs.GradientSync(comm, bucket, True)

    def run(m, *extra):
        if amp:
            with cs.autocast(s, torch.bfloat16):
                return m.forward_loss(s, T(x), T(y))
        return m.forward_loss(s, T(x), T(y))

    loss_tp = run(tp)
    tp.backward_loss(s, sync)
    bucket.sync(s, comm)
    loss_full = run(full)
    full.backward_loss(s)
    s.synchronize()
    lt = cs.to_torch(s, loss_tp).double().to("cpu")
    gathered = [torch.zeros_like(lt) for _ in range(world)]
    dist.all_gather(gathered, lt) if device == "cpu" else None
    if device == "cpu":
        assert abs(sum(gathered).item() / world - loss_full.raw().item()) < 1e-9
    if expect_fused:
        assert C.fused_tp_launches() >= 16, C.fused_tp_launches()  # per block: 2 gathers + 2 reduce-scatters forward and backward
        lf, ltp = loss_full.raw().item(), cs.to_torch(s, loss_tp).item()
        assert abs(lf - ltp) < 0.2, (lf, ltp)
    gt, gf = tp.named_gradients(), full.named_gradients()
    tol = dict(atol=3e-2, rtol=5e-2) if amp else dict(atol=1e-9, rtol=1e-7)
    for k, gtp in gt.items():
        ref = full_grad_slice(k, gf[full_key(k)].raw(), rank, world, cfg)
        got = gtp.raw() / world
        if amp:
            err = (got.float() - ref.float()).norm() / (ref.float().norm() + 1e-12)
            assert err < 6e-2, (rank, k, err.item())
        else:
            assert torch.allclose(got, ref, **tol), (rank, k, (got - ref).abs().max().item())


def case_tp_checkpoint_merge(device, nvp2p):
    """Per-rank parameter files of a tensor-parallel model (uneven heads: 3 over 2 ranks) unite into a file that the
    unsharded model loads, and that model then computes the tensor-parallel ranks' mean loss."""
    import shutil

    from core_scheduler_b200.utils.checkpoint import merge_tensor_parallel, read_parameters, write_parameters

    comm, rank, world, s = make_comm(device, nvp2p)
    cs.manual_seed(23 + rank)  # the ranks' own shards must differ for the test to mean anything
    cfg = cs.GPT2Config(n_layer=2, n_head=3, n_embd=48, block_size=32, vocab_size=128, padded_vocab_size=128, dtype=torch.float64)
    tp = C.TPGPT2(s, cfg, comm)
    replicated = tp.replicated_parameters()
    for k, p in tp.named_parameters().items():  # replicated parameters have to agree across the ranks
        if k in replicated:
            dist.broadcast(p.raw(), src=0)
    directory = f"/tmp/cs_tp_merge_{os.environ.get('MASTER_PORT', '0')}"
    os.makedirs(f"{directory}/tp_rank{rank}", exist_ok=True)
    tp.save(f"{directory}/tp_rank{rank}/model.parquet")
    dist.barrier()
    merged = merge_tensor_parallel([read_parameters(f"{directory}/tp_rank{r}/model.parquet") for r in range(world)], cfg.n_head, cfg.n_embd)
    write_parameters(merged, f"{directory}/model.rank{rank}.parquet")
    cs.manual_seed(99)
    full = cs.GPT2(s, cfg)
    full.load(f"{directory}/model.rank{rank}.parquet")  # unknown or missing keys would raise
    fp = full.named_parameters()
    for k, p in tp.named_parameters().items():
        mine = tp_slice(k, fp[full_key(k)].raw(), rank, world, cfg)
        assert torch.allclose(mine, p.raw(), atol=1e-6), (rank, k)  # the file holds float32 values
    ids = torch.randint(0, 128, (2 * world, 33), generator=torch.Generator().manual_seed(29))
    x, y = T(ids[:, :-1].contiguous()), T(ids[:, 1:].contiguous())
    mine = tp.forward_loss(s, x, y).raw().double().reshape(1)
    parts = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    whole = full.forward_loss(s, x, y).raw().item()
    assert abs(sum(p.item() for p in parts) / world - whole) < 1e-5, (parts, whole)
    dist.barrier()
    if rank == 0:
        shutil.rmtree(directory, ignore_errors=True)


def case_watchdog(device, nvp2p):
    """A rank whose loop stalls trips its watchdog; the healthy rank learns of it through the store before its next launch."""
    comm, rank, world, s = make_comm(device, False)
    dog = C.Watchdog(comm, timeout_ms=300, poll_ms=20)
    for step in range(3):
        dog.progress(step)
        dog.check()
        time.sleep(0.05)
    dist.barrier()
    if rank == world - 1:
        time.sleep(1.0)  # the stall: no progress() calls
        assert dog.tripped() and dog.last_step() == 2
    else:
        deadline = time.time() + 10
        while time.time() < deadline and not dog.failed_peers():
            dog.progress(3)
            time.sleep(0.05)
        assert dog.failed_peers() == [world - 1], dog.failed_peers()
        assert not dog.tripped()
        try:
            dog.check()
            raised = False
        except RuntimeError as e:
            raised = "reported a failure" in str(e)
        assert raised
    dog.stop()
    dist.barrier()


def case_failure_injection(device, nvp2p):
    """A collective that fails on one rank surfaces as an error there; the others see the rank stop beating."""
    comm, rank, world, s = make_comm(device, False)
    hb = C.Heartbeat(comm, 500)
    hb.beat(0)
    dist.barrier()
    assert hb.stale_ranks() == []
    x = T(torch.ones(8, device=device))
    C.all_reduce(s, comm, [x], "sum")  # healthy step
    failed = False
    if rank == world - 1:
        comm.inject_failure_after(0)
        try:
            C.all_reduce(s, comm, [x], "sum")
        except RuntimeError as e:
            failed = "injected communication failure" in str(e)
        assert failed
        # this rank stops between steps (nothing in flight) and never beats again
    else:
        deadline = time.time() + 10
        stale = []
        while time.time() < deadline:
            hb.beat(1)
            stale = hb.stale_ranks()
            if stale:
                break
            time.sleep(0.1)
        assert stale == [world - 1], (rank, stale)
    dist.barrier()


def case_timeout_status(device, nvp2p):
    """A peer flag that nothing sets: the barrier kernel gives up within its budget and reports it."""
    comm, rank, world, s = make_comm(device, True)
    ctx = C.create_symmetric_context(comm, 1 << 20)
    C.set_peer_wait_budget(2_000_000)  # about a millisecond
    if rank == 0:
        C.symmetric_barrier(s, comm)   # nobody else joins this barrier
        s.synchronize()
        try:
            ctx.check_status()
            raised = False
        except RuntimeError as e:
            raised = "timed out" in str(e)
        assert raised
        ctx.check_status()  # cleared, context still usable
        y = torch.ones(4, device="cuda") * 2
        assert y.sum().item() == 8
    dist.barrier()
    C.set_peer_wait_budget(4_000_000_000)


CASES = {k[len("case_"):]: v for k, v in globals().items() if k.startswith("case_")}

if __name__ == "__main__":
    device, case = sys.argv[1], sys.argv[2]
    nvp2p = len(sys.argv) > 3 and sys.argv[3] == "nvp2p"
    CASES[case](device, nvp2p)
    if dist.is_initialized():
        dist.barrier()
        if dist.get_rank() == 0:
            print(f"OK {case}")
        dist.destroy_process_group()
    else:
        print(f"OK {case}")
