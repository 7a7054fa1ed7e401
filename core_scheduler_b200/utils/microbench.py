# SPDX-License-Identifier: Apache-2.0
"""Kernel microbenchmarks with CUDA-event timing (after warm-up, L2 flushed between iterations).

  python -m core_scheduler_b200.utils.microbench gemm        # tcgen05 GEMM vs torch.matmul (cuBLAS)
  python -m core_scheduler_b200.utils.microbench elementwise # LayerNorm / GELU / AdamW bandwidth
  python -m core_scheduler_b200.utils.microbench attention    # tcgen05 attention forward vs cuDNN
  python -m core_scheduler_b200.utils.microbench kernels_once # every non-GEMM kernel twice (profiler workload)
  python -m core_scheduler_b200.utils.microbench collectives_loopback [ranks] [MiB]
                                                              # collective and fused GEMM+collective kernels of ONE emulated
                                                              # rank on one GPU (peer memory = local memory): profiler workload

Prints one line per case: achieved TFLOP/s or GB/s and the fraction of the measured peak
(MEASURED_PEAKS.json at the repository root when present, else the fallback 1.59 PFLOP/s, 6.65 TB/s).
"""
from __future__ import annotations

import json
import os
import sys

import torch

import core_scheduler_b200 as cs

C = cs._C
BF = torch.bfloat16
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, iters=10, warmup=3, stream=None):
    """Median CUDA-event time of fn() on `stream` (the launching stream; default: torch's current)."""
    stream = stream or torch.cuda.current_stream()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush_l2()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def bench_gemm():
    tflops_peak, _, tag = peaks()
    shapes = [  # (name, layout, M, N, K) in GEMM terms; GPT-2 124M at 16x1024 tokens
        ("c_attn fwd", 0, 16384, 2304, 768), ("c_proj fwd", 0, 16384, 768, 768), ("fc1 fwd", 0, 16384, 3072, 768),
        ("fc2 fwd", 0, 16384, 768, 3072), ("lm_head fwd", 0, 16384, 50304, 768), ("lm_head dgrad", 0, 16384, 768, 50304),
        ("fc1 wgrad", 1, 3072, 768, 16384), ("c_attn wgrad", 1, 2304, 768, 16384), ("c_proj wgrad", 1, 768, 768, 16384),
        ("lm_head wgrad", 1, 50304, 768, 16384), ("square 8192", 0, 8192, 8192, 8192),
    ]
    for name, layout, M, N, K in shapes:
        if layout == 0:
            a = torch.randn(M, K, device="cuda").to(BF)
            b = torch.randn(N, K, device="cuda").to(BF)
            d = torch.empty(M, N, device="cuda", dtype=BF)
            ours = lambda: C.gemm_bf16(a, b, d, 0, 0)
            lib = lambda: torch.matmul(a, b.t(), out=d)
        else:
            a = torch.randn(K, M, device="cuda").to(BF)
            b = torch.randn(K, N, device="cuda").to(BF)
            d = torch.empty(M, N, device="cuda")
            d16 = torch.empty(M, N, device="cuda", dtype=BF)
            ours = lambda: C.gemm_bf16(a, b, d, 1, 4)
            lib = lambda: torch.matmul(a.t(), b, out=d16)
        flops = 2.0 * M * N * K
        t_ours, t_lib = time_ms(ours), time_ms(lib)
        print(f"gemm {name:14s} M={M:6d} N={N:6d} K={K:6d}  ours {t_ours:8.4f} ms {flops / t_ours / 1e9:8.1f} TFLOP/s "
              f"({flops / t_ours / 1e9 / tflops_peak:.2f} of {tag})   cuBLAS {t_lib:8.4f} ms {flops / t_lib / 1e9:8.1f} TFLOP/s")


def bench_elementwise():
    _, gbs_peak, tag = peaks()
    s = cs.DynamicScheduler(0, device="cuda")
    main = torch.cuda.ExternalStream(s.raw_stream(0))
    assist = torch.cuda.ExternalStream(s.raw_stream(1))
    rows, d = 16384, 768
    x = torch.randn(rows, d, device="cuda").to(BF)
    ln = C.layer_norm_init(s, [d])
    tx = cs.from_torch(x)

    def ln_fwd():
        with cs.autocast(s, BF):
            C.layer_norm_forward(s, ln, tx)

    t = time_ms(ln_fwd, stream=main)
    print(f"layernorm fwd [{rows},{d}] {t:.4f} ms {2 * x.numel() * 2 / t / 1e6:.0f} GB/s ({2 * x.numel() * 2 / t / 1e6 / gbs_peak:.2f} of {tag})")
    dy = cs.from_torch(torch.randn(rows, d, device="cuda").to(BF))

    def ln_bwd():
        with cs.autocast(s, BF):
            C.layer_norm_forward(s, ln, tx)
        C.layer_norm_backward(s, ln, dy, dy)

    t_both = time_ms(ln_bwd, stream=main)
    print(f"layernorm fwd+bwd(+residual) [{rows},{d}] {t_both:.4f} ms -> bwd alone {t_both - t:.4f} ms "
          f"{4 * x.numel() * 2 / (t_both - t) / 1e6:.0f} GB/s ({4 * x.numel() * 2 / (t_both - t) / 1e6 / gbs_peak:.2f} of {tag})")
    g = C.gelu_init(s)
    y = torch.randn(rows, 4 * d, device="cuda").to(BF)
    ty = cs.from_torch(y)
    t = time_ms(lambda: C.gelu_forward(s, g, ty), stream=main)
    print(f"gelu fwd [{rows},{4 * d}] {t:.4f} ms {2 * y.numel() * 2 / t / 1e6:.0f} GB/s ({2 * y.numel() * 2 / t / 1e6 / gbs_peak:.2f} of {tag})")
    n = 163_000_000
    w = cs.from_torch(torch.randn(n, device="cuda"))
    C.working_copy(s, w, BF)
    st = C.adamw_init(s, w)
    gr = cs.from_torch(torch.randn(n, device="cuda"))
    t = time_ms(lambda: C.adamw_step(s, st, w, gr), stream=assist)
    bytes_moved = n * (4 * 4 + 3 * 4 + 2)
    print(f"adamw fp32 master + bf16 copy n={n} {t:.4f} ms {bytes_moved / t / 1e6:.0f} GB/s ({bytes_moved / t / 1e6 / gbs_peak:.2f} of {tag})")


def bench_attention():
    """tcgen05 causal attention forward and backward vs the cuDNN engine, GPT-2 124M shape (B16 H12 T1024 D64)."""
    tflops_peak, _, tag = peaks()
    B, T, H, D = 16, 1024, 12, 64
    qkv = torch.randn(B, T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(B, T, H * D, device="cuda").to(BF)
    scale = D ** -0.5
    ours = lambda: C.attention_forward_tcgen05(qkv, H, scale)
    q, k, v = (x.transpose(1, 2) for x in qkv.view(B, T, 3, H, D).unbind(2))
    lib = lambda: torch.ops.aten._scaled_dot_product_cudnn_attention(q, k, v, None, True, 0.0, True, False, scale=scale)
    flops = 4.0 * B * H * T * T * D / 2  # causal
    t_ours, t_lib = time_ms(ours), time_ms(lib)
    print(f"attention fwd causal B={B} H={H} T={T} D={D}: ours {t_ours * 1e3:.1f} us {flops / t_ours / 1e9:.0f} TFLOP/s "
          f"({flops / t_ours / 1e9 / tflops_peak:.2f} of {tag})   cuDNN {t_lib * 1e3:.1f} us {flops / t_lib / 1e9:.0f} TFLOP/s   "
          f"status {C.attention_status()}")
    _, out, lse = ours()
    ours_bwd = lambda: C.attention_backward_tcgen05(qkv, out, dout, lse, H, scale)
    qa, ka, va = (x.detach().requires_grad_(True) for x in (q, k, v))
    o_lib = torch.nn.functional.scaled_dot_product_attention(qa, ka, va, is_causal=True, scale=scale)
    go = dout.view(B, T, H, D).transpose(1, 2)

    def lib_bwd():
        torch.autograd.grad(o_lib, (qa, ka, va), go, retain_graph=True)

    with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.CUDNN_ATTENTION):
        o_lib = torch.nn.functional.scaled_dot_product_attention(qa, ka, va, is_causal=True, scale=scale)
        t_lib_b = time_ms(lib_bwd)
    t_ours_b = time_ms(ours_bwd)
    fb = 2.5 * flops  # five matrix products in the minimal backward
    print(f"attention bwd causal (3 launches: delta, dK/dV, dQ): ours {t_ours_b * 1e3:.1f} us {fb / t_ours_b / 1e9:.0f} TFLOP/s "
          f"(useful; the kernels run 7 products) ({fb / t_ours_b / 1e9 / tflops_peak:.2f} of {tag})   cuDNN {t_lib_b * 1e3:.1f} us "
          f"{fb / t_lib_b / 1e9:.0f} TFLOP/s   status {C.attention_status()}")


def collectives_loopback():
    """One launch of every peer-memory kernel as rank 0 of `ranks` emulated ranks on this GPU (all arenas local, peer
    flags primed): what a profiler can capture of these kernels without a second process. Times are those of the
    kernel's own memory traffic on local HBM (no NVLink): every peer load and store is a local one."""
    ranks = int(sys.argv[2]) if len(sys.argv) > 2 else 2
    mib = int(sys.argv[3]) if len(sys.argv) > 3 else 256
    _, gbs_peak, tag = peaks()
    n = (mib << 20) // 4
    ctxs = C.create_loopback_contexts(ranks, 3 * (mib << 20) + (256 << 20) * 2)
    ctx = ctxs[0]
    stream = torch.cuda.current_stream()

    def run(name, fn, nbytes):
        for _ in range(2):
            ctx.prime_loopback()
            fn()
        torch.cuda.synchronize()
        ctx.prime_loopback()
        flush_l2()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        torch.cuda.synchronize()
        t = a.elapsed_time(b)
        ctx.check_status()
        print(f"{name:58s} {t * 1e3:9.1f} us  {nbytes / t / 1e6:7.0f} GB/s of local traffic ({nbytes / t / 1e6 / gbs_peak:.2f} of {tag} copy bandwidth)", flush=True)

    grads = [c.empty([n], torch.float32)[0] for c in ctxs]
    for g in grads:
        g.normal_()
    # rank 0 reduces its 1/ranks slice: reads it from every rank, writes it to every rank
    run(f"all_reduce fp32 {mib} MiB, {ranks} ranks (rank 0's slice)", lambda: ctx.all_reduce_([grads[0]], "sum"), 2 * (mib << 20))
    half = [c.empty([ranks, n // ranks // 2], BF)[0] for c in ctxs]
    out = torch.empty(n // ranks // 2, device="cuda", dtype=BF)
    run("reduce_scatter bf16 (rank 0's chunk from every rank)", lambda: ctx.reduce_scatter_(out, [half[0][p] for p in range(ranks)], "sum"),
        (ranks + 1) * out.numel() * 2)
    shard = torch.randn(n // ranks // 2, device="cuda").to(BF)
    run("all_gather bf16 push (rank 0's shard to every rank)", lambda: ctx.all_gather_([half[0][p] for p in range(ranks)], shard),
        (ranks + 1) * shard.numel() * 2)
    lps = [c.empty([n], BF)[0] for c in ctxs]
    block = C.ZeroAdamW.block
    per = ((n + block - 1) // block + ranks - 1) // ranks * block
    w, m, v = (torch.zeros(per, device="cuda") for _ in range(3))
    run("reduce-scatter + AdamW + all-gather (rank 0's blocks)", lambda: ctx.sharded_adamw_(grads[0], lps[0], w, m, v, 0, n, block, 1e-3, 0.9, 0.95,
                                                                                            1e-8, 0.1, 1, 1.0 / ranks),
        n // ranks * (4 * ranks + 6 * 4 + 2 * ranks))
    # tensor-parallel pair: rows gathered in chunks beside the GEMM that consumes them; GEMM with the scatter in its epilogue
    rows, k, nn = 4096, 1280, 640
    fulls = [c.empty([ranks * rows, k], BF)[0] for c in ctxs]
    xs = torch.randn(rows, k, device="cuda").mul_(0.5).to(BF)
    wt = torch.randn(nn, k, device="cuda").mul_(0.05).to(BF)
    sig = [None]

    def gather():
        sig[0] = ctx.gather_rows_chunked(xs, fulls[0], 4)

    run(f"gather rows in 4 chunks [{rows},{k}] x {ranks} ranks", gather, (ranks + 1) * xs.numel() * 2)
    run(f"GEMM on gathered chunks [{ranks * rows},{k}] x [{nn},{k}]^T", lambda: ctx.gemm_on_gathered_chunks(fulls[0], wt, False, 0, None, sig[0]),
        fulls[0].numel() * 2 + ranks * rows * nn * 2)
    slots = [c.empty([ranks, rows, k], BF)[0] for c in ctxs]
    xa = torch.randn(ranks * rows, nn, device="cuda").mul_(0.5).to(BF)
    w2 = torch.randn(k, nn, device="cuda").mul_(0.05).to(BF)
    run(f"GEMM with scatter epilogue [{ranks * rows},{nn}] x [{k},{nn}]^T", lambda: ctx.gemm_scatter_to_slots(xa, w2, False, slots[0]),
        xa.numel() * 2 + ranks * rows * k * 2)
    res = torch.randn(rows, k, device="cuda").to(BF)
    run(f"slot sum + residual [{ranks},{rows},{k}]", lambda: ctx.sum_slots(slots[0], res), (ranks + 2) * rows * k * 2)
    print("gemm status", C.gemm_status())


def gemm_one():
    """One GPT-2 shape (fc1), a handful of launches: the workload for an ncu capture.

    Optional argument: epilogue id (0 store, 1 residual, 2 GELU dual, 3 dGELU)."""
    epi = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    M, N, K = 16384, 3072, 768
    a = torch.randn(M, K, device="cuda").to(BF)
    b = torch.randn(N, K, device="cuda").to(BF)
    d = torch.empty(M, N, device="cuda", dtype=BF)
    aux = torch.randn(M, N, device="cuda").to(BF) if epi in (1, 3) else None
    d2 = torch.empty_like(d) if epi == 2 else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(6):
        if i == 3:
            start.record()
        C.gemm_bf16(a, b, d, 0, epi, aux=aux, d2=d2)
    stop.record()
    torch.cuda.synchronize()
    print(f"gemm_one epilogue={epi}: {start.elapsed_time(stop) / 3 * 1e3:.1f} us per launch")


def kernels_once():
    """Every non-GEMM kernel of the training step, twice each on inputs larger than L2 (a few GB in
    total): the workload for a profiler capture and a per-kernel bandwidth table (second launch timed)."""
    _, gbs_peak, tag = peaks()
    s = cs.DynamicScheduler(0, device="cuda")
    main = torch.cuda.ExternalStream(s.raw_stream(0))
    rows, d, V = 65536, 768, 50304
    T = cs.from_torch

    def run(name, fn, nbytes, stream=None):
        stream = stream or main
        fn()
        s.synchronize()
        flush_l2()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        s.synchronize()
        torch.cuda.synchronize()
        t = a.elapsed_time(b)
        print(f"{name:34s} {t * 1e3:9.1f} us  {nbytes / t / 1e6:7.0f} GB/s ({nbytes / t / 1e6 / gbs_peak:.2f} of {tag} copy bandwidth)", flush=True)

    x = torch.randn(rows, d, device="cuda").to(BF)
    dy = torch.randn(rows, d, device="cuda").to(BF)
    ln = C.layer_norm_init(s, [d])

    def ln_fwd():
        with cs.autocast(s, BF):
            C.layer_norm_forward(s, ln, T(x))

    run("layernorm fwd [65536,768]", ln_fwd, 2 * x.numel() * 2)
    # backward of the pre-norm block: dx = LN'(dy) + residual gradient, dgamma/dbeta partials

    def ln_fwd_bwd():  # backward consumes the state its forward saved, so the pair runs together
        ln_fwd()
        C.layer_norm_backward(s, ln, T(dy), T(dy))

    run("layernorm fwd + bwd(+residual)", ln_fwd_bwd, 6 * x.numel() * 2)
    g = C.gelu_init(s)
    h = torch.randn(rows // 2, 4 * d, device="cuda").to(BF)
    run("gelu fwd [32768,3072]", lambda: C.gelu_forward(s, g, T(h)), 2 * h.numel() * 2)

    def gelu_fwd_bwd():
        C.gelu_forward(s, g, T(h))
        C.gelu_backward(s, g, T(h))

    run("gelu fwd + bwd", gelu_fwd_bwd, 5 * h.numel() * 2)
    run("add bf16", lambda: C.utils_add(s, T(h), T(h)), 3 * h.numel() * 2)
    n = 32 << 20
    w = T(torch.randn(n, device="cuda"))
    C.working_copy(s, w, BF)
    st = C.adamw_init(s, w)
    gr = T(torch.randn(n, device="cuda"))
    assist = torch.cuda.ExternalStream(s.raw_stream(1))
    run("adamw fp32 master -> bf16 copy 32M", lambda: C.adamw_step(s, st, w, gr), n * (4 * 4 + 3 * 4 + 2), assist)
    te, pe = C.embedding_init(s, V, d), C.embedding_init(s, 1024, d)
    idx = torch.randint(0, 50257, (64, 1024), device="cuda")
    dye = dy.view(64, 1024, d)

    def emb_fwd():
        with cs.autocast(s, BF):
            C.embedding_forward_token_position(s, te, pe, T(idx))

    run("embedding fwd (token+position)", emb_fwd, 2 * dye.numel() * 2)

    def emb_fwd_bwd():
        emb_fwd()
        C.embedding_backward_token_position(s, te, pe, T(dye))

    run("embedding fwd + bwd (token+position)", emb_fwd_bwd, 3 * dye.numel() * 2 + 2 * dye.numel() * 4)
    norm_in = [T(torch.randn(n, device="cuda"))]
    run("grad-norm + clip 32M fp32", lambda: C.utils_clip_grad_norm_(s, norm_in, 1.0), n * 4 * 3)
    B, Tn, H, D = 16, 1024, 12, 64
    qkv = torch.randn(B, Tn, 3 * H * D, device="cuda").to(BF)
    run("attention fwd tcgen05 B16 H12 T1024", lambda: C.attention_forward_tcgen05(qkv, H, D ** -0.5), 4 * B * Tn * H * D * 2,
        torch.cuda.current_stream())
    lin = C.linear_init(s, d, V, bias=False)
    ce = C.linear_cross_entropy_init(s, lin, valid_classes=50257)
    xs = torch.randn(8192, d, device="cuda").to(BF)
    tg = torch.randint(0, 50257, (8192,), device="cuda")

    def ce_fwd_bwd():
        with cs.autocast(s, BF):
            C.linear_cross_entropy_forward(s, ce, T(xs), T(tg))
        C.linear_cross_entropy_backward(s, ce)

    run("classifier+cross-entropy fwd+bwd 8192", ce_fwd_bwd, 3 * 8192 * V * 2)
    print("attention status", C.attention_status(), "gemm status", C.gemm_status())


if __name__ == "__main__":
    import json

    from core_scheduler_b200.utils.clocks import ClockSampler

    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    sampler = ClockSampler(torch.cuda.current_device()).start()  # read-only; every table ends with its clock record
    try:
        {"gemm": bench_gemm, "elementwise": bench_elementwise, "gemm_one": gemm_one, "attention": bench_attention,
         "kernels_once": kernels_once, "collectives_loopback": collectives_loopback}[what]()
    finally:
        print("clocks during the run:", json.dumps(sampler.stop()), flush=True)
