# SPDX-License-Identifier: Apache-2.0
"""AdamW, module tree naming, flat arenas, checkpoints."""
import os

import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

import core_scheduler_b200 as cs
from helpers import T

C = cs._C


def adamw_reference(w, g, m, v, t, lr, b1, b2, eps, wd, vmax=None):
    w = w - lr * wd * w
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    mh = m / (1 - b1**t)
    vh = v / (1 - b2**t)
    if vmax is not None:
        vmax = torch.maximum(vmax, vh)
        vh = vmax
    w = w - lr * mh / (vh.sqrt() + eps)
    return w, m, v, vmax


@pytest.mark.parametrize("n", [128, 512, 1024])
@pytest.mark.parametrize("amsgrad", [False, True])
def test_functional_adamw_matches_formula(cpu_scheduler, n, amsgrad):
    s = cpu_scheduler
    w0 = torch.randn(n)
    w = T(w0.clone())
    st = C.adamw_init(s, w, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, amsgrad=amsgrad)
    wr, m, v = w0.clone(), torch.zeros(n), torch.zeros(n)
    vmax = torch.zeros(n) if amsgrad else None
    for t in range(1, 4):
        g = torch.randn(n)
        C.adamw_step(s, st, w, T(g))
        wr, m, v, vmax = adamw_reference(wr, g, m, v, t, 1e-2, 0.9, 0.95, 1e-8, 0.1, vmax)
    assert torch.allclose(w.raw(), wr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(st.m.raw(), m, rtol=1e-4, atol=1e-6)
    assert torch.allclose(st.v.raw(), v, rtol=1e-4, atol=1e-6)


def test_module_adamw_matches_torch_optim(cpu_scheduler):
    s = cpu_scheduler
    lin = C.LinearModule(s, 16, 8, bias=True)
    ref = torch.nn.Linear(16, 8)
    with torch.no_grad():
        ref.weight.copy_(lin.state().weight.raw())
        ref.bias.copy_(lin.state().bias.raw())
    opt = cs.AdamW(s, lin, lr=1e-2, weight_decay=0.05)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.05)
    for _ in range(3):
        x, dy = torch.randn(4, 16), torch.randn(4, 8)
        lin.forward(s, T(x))
        lin.backward(s, T(dy))
        opt.step(s)
        opt.zero_grad(s)
        ropt.zero_grad()
        ref(x).backward(dy)
        ropt.step()
    assert torch.allclose(lin.state().weight.raw(), ref.weight, rtol=1e-4, atol=1e-5)
    assert torch.allclose(lin.state().bias.raw(), ref.bias, rtol=1e-4, atol=1e-5)
    opt.set_lr(0.5)
    assert opt.get_lr() == 0.5


def test_amp_adamw_updates_master_and_working_copy(cpu_scheduler):
    s = cpu_scheduler
    w32 = T(torch.randn(64))
    w16 = T(w32.raw().bfloat16())
    st = C.adamw_init(s, w32, lr=1e-2)
    g = torch.randn(64).bfloat16()
    C.amp_adamw_step(s, st, w16, w32, T(g))
    wr, _, _, _ = adamw_reference(w16.raw().float() * 0 + w32.raw() * 0 + w32.raw(), g.float(), 0, 0, 1, 1e-2, 0.9, 0.999, 1e-8, 1e-2)
    assert w16.raw().dtype == torch.bfloat16 and torch.equal(w16.raw(), w32.raw().bfloat16())


def test_gpt2_parameter_names_follow_reference_layout(cpu_scheduler):
    cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=32, block_size=16, vocab_size=64, padded_vocab_size=64)
    m = cs.GPT2(cpu_scheduler, cfg)
    names = m.parameter_names()
    assert names[:2] == ["wte.weight", "wpe.weight"]
    assert names[2:10] == [
        "0.ln1.weight", "0.ln1.bias", "0.attn.c_attn.weight", "0.attn.c_proj.weight",
        "0.ln2.weight", "0.ln2.bias", "0.mlp.fc1.weight", "0.mlp.fc2.weight",
    ]
    assert names[-3:] == ["lnf.weight", "lnf.bias", "lm_head.weight"]
    total = sum(p.numel() for p in m.named_parameters().values())
    assert total == cfg.parameter_count()


def test_standalone_module_has_empty_prefix(cpu_scheduler):
    ln = C.LayerNormModule(cpu_scheduler, 8)
    assert ln.parameter_names() == [".weight", ".bias"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_save_load_round_trip_and_schema(cpu_scheduler, tmp_path, dtype):
    s = cpu_scheduler
    ln = C.LayerNormModule(s, 384, dtype=dtype)
    ln.state().weight.raw().uniform_(-1, 1)
    ln.state().bias.raw().uniform_(-1, 1)
    keep_w, keep_b = ln.state().weight.raw().clone(), ln.state().bias.raw().clone()
    path = str(tmp_path / "model.parquet")
    ln.save(path)
    table = pq.read_table(path)
    assert table.schema.names == ["key", "value"]
    assert str(table.schema.field("key").type) == "string"
    vt = table.schema.field("value").type
    assert pa.types.is_list(vt) and vt.value_type == pa.float32()
    assert table.column("key").to_pylist() == [".weight", ".bias"]
    ln.state().weight.raw().zero_()
    ln.state().bias.raw().zero_()
    ln.load(path)
    assert torch.allclose(ln.state().weight.raw(), keep_w.float().to(dtype))
    assert torch.allclose(ln.state().bias.raw(), keep_b.float().to(dtype))


def test_load_rejects_unknown_keys(cpu_scheduler, tmp_path):
    a = C.LayerNormModule(cpu_scheduler, 8)
    b = C.LinearModule(cpu_scheduler, 8, 8)
    path = str(tmp_path / "a.parquet")
    a.save(path)
    a.load(path)
    pq.write_table(pa.table({"key": ["nope.weight"], "value": [[1.0, 2.0]]}), path)
    with pytest.raises(RuntimeError):
        b.load(path)


def test_optimizer_checkpoint_round_trip(cpu_scheduler, tmp_path):
    s = cpu_scheduler
    lin = C.LinearModule(s, 8, 4, bias=False)
    opt = cs.AdamW(s, lin, lr=1e-2)
    lin.forward(s, T(torch.randn(3, 8)))
    lin.backward(s, T(torch.randn(3, 4)))
    opt.step(s)
    path = str(tmp_path / "opt.parquet")
    opt.save(path)
    m = opt.named_state_tensors()[".weight.m"].raw().clone()
    opt.named_state_tensors()[".weight.m"].raw().zero_()
    opt2 = cs.AdamW(s, lin, lr=5.0)
    opt2.load(path)
    assert torch.allclose(opt2.named_state_tensors()[".weight.m"].raw(), m)
    assert opt2.step_count() == 1 and abs(opt2.get_lr() - 1e-2) < 1e-9


def test_flat_arenas_preserve_values_and_make_gradients_persistent(cpu_scheduler):
    s = cpu_scheduler
    cfg = cs.GPT2Config(n_layer=1, n_head=2, n_embd=32, block_size=16, vocab_size=64, padded_vocab_size=64)
    m = cs.GPT2(s, cfg)
    before = {k: v.raw().clone() for k, v in m.named_parameters().items()}
    flat = C.flatten_parameters(s, m, lp_dtype=torch.bfloat16)
    after = m.named_parameters()
    for k, v in before.items():
        assert torch.equal(after[k].raw(), v)
        assert after[k].raw().untyped_storage().data_ptr() == flat.params.raw().untyped_storage().data_ptr()
        assert after[k].lp().dtype == torch.bfloat16
    for key, off, n in flat.slots():
        assert off % 128 == 0
    ids = torch.randint(0, 64, (2, 16))
    loss = m.forward_loss(s, T(ids), T(torch.roll(ids, -1, 1)))
    m.backward_loss(s)
    g = m.named_gradients()["lm_head.weight"]
    assert g.is_persistent() and not g.is_fresh()
    assert g.raw().untyped_storage().data_ptr() == flat.grads.raw().untyped_storage().data_ptr()
    m.zero_grad()
    assert g.defined() and g.is_fresh()
    del loss


def test_flat_adamw_equals_per_tensor_adamw(cpu_scheduler):
    s = cpu_scheduler
    cfg = cs.GPT2Config(n_layer=1, n_head=2, n_embd=32, block_size=16, vocab_size=64, padded_vocab_size=64)
    cs.manual_seed(5)
    a = cs.GPT2(s, cfg)
    cs.manual_seed(5)
    b = cs.GPT2(s, cfg)
    flat = C.flatten_parameters(s, b)
    oa = cs.AdamW(s, a, lr=1e-2, weight_decay=0.1)
    ob = cs.AdamW(s, b, lr=1e-2, weight_decay=0.1, flat=flat)
    for i in range(3):
        ids = torch.randint(0, 64, (2, 16))
        lab = torch.roll(ids, -1, 1)
        la = a.forward_loss(s, T(ids), T(lab)); a.backward_loss(s); oa.step(s); oa.zero_grad(s)
        lb = b.forward_loss(s, T(ids), T(lab)); b.backward_loss(s); ob.step(s); ob.zero_grad(s)
        assert torch.allclose(la.raw(), lb.raw(), atol=1e-5)
    pa, pb = a.named_parameters(), b.named_parameters()
    for k in pa:
        assert torch.allclose(pa[k].raw(), pb[k].raw(), atol=1e-5), k


def test_flat_arenas_lay_named_parameters_out_first(cpu_scheduler):
    """`first=` puts a group of parameters ahead of the others, in the given order and without gaps beyond slot
    padding; values survive, training is unchanged, an unknown name is refused."""
    s = cpu_scheduler
    cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=32, block_size=16, vocab_size=64, padded_vocab_size=64)
    cs.manual_seed(6)
    a = cs.GPT2(s, cfg)
    cs.manual_seed(6)
    b = cs.GPT2(s, cfg)
    group = ["lnf.bias", "1.ln2.weight", "wpe.weight", "0.ln1.bias"]
    before = {k: v.raw().clone() for k, v in b.named_parameters().items()}
    flat = C.flatten_parameters(s, b, first=group)
    slots = flat.slots()
    assert [k for k, _, _ in slots[:len(group)]] == group
    rest = [k for k in a.named_parameters().keys() if k not in group]
    assert [k for k, _, _ in slots[len(group):]] == rest  # module order otherwise
    end = 0
    for key, off, n in slots:
        assert off == end  # consecutive slots: a group is one range
        end = off + (n + 127) // 128 * 128
    for k, v in before.items():
        assert torch.equal(b.named_parameters()[k].raw(), v)
    oa = cs.AdamW(s, a, lr=1e-2, weight_decay=0.1, flat=C.flatten_parameters(s, a))
    ob = cs.AdamW(s, b, lr=1e-2, weight_decay=0.1, flat=flat)
    for i in range(2):
        ids = torch.randint(0, 64, (2, 16))
        lab = torch.roll(ids, -1, 1)
        la = a.forward_loss(s, T(ids), T(lab)); a.backward_loss(s); oa.step(s); oa.zero_grad(s)
        lb = b.forward_loss(s, T(ids), T(lab)); b.backward_loss(s); ob.step(s); ob.zero_grad(s)
        assert torch.equal(la.raw(), lb.raw())
    for k, v in a.named_parameters().items():
        assert torch.equal(v.raw(), b.named_parameters()[k].raw()), k
    with pytest.raises(Exception, match="not a parameter"):
        C.flatten_parameters(s, cs.GPT2(s, cfg), first=["no.such.weight"])


def test_symmetric_arena_offsets_coalesce_and_return_to_the_top():
    """The peer-mapped arena hands out offsets; freed neighbours unite, so growing requests keep fitting."""
    ctx = cs._C.SymmetricContext(arena_bytes=1 << 20)
    a, b, c = (ctx.allocate(n) for n in (1000, 5000, 300))
    assert a == (0, 1024) and b == (1024, 5120) and c == (6144, 512)
    ctx.release(*a)
    ctx.release(*b)  # unites with a: one cached block of 6144 bytes
    assert ctx.cached_blocks() == 1
    d = ctx.allocate(6000)
    assert d == (0, 6144) and ctx.cached_blocks() == 0
    e = ctx.allocate(256)
    assert e[0] == 6656
    ctx.release(*e)  # top of the arena: goes back to the bump pointer
    assert ctx.cached_blocks() == 0 and ctx.allocate(512)[0] == 6656
    # doubling sizes with release in between never exhaust an arena of 3x the largest request
    small = cs._C.SymmetricContext(arena_bytes=3 << 20)
    size = 1024
    while size <= (1 << 20):
        x, y = small.allocate(size), small.allocate(size)
        small.release(*x)
        small.release(*y)
        size *= 2
    assert small.bytes_in_use() == 0
    with pytest.raises(RuntimeError, match="exhausted"):
        small.allocate(4 << 20)
    f = small.allocate(100)
    g = small.allocate(100)
    small.release(*f)
    h = small.allocate(50)  # best fit splits nothing smaller than the alignment
    assert h == f and g[0] == 256


def test_symmetric_arena_random_sequences_never_overlap_and_fully_coalesce():
    """Property test of the offset allocator: live blocks are disjoint, aligned and inside the arena whatever the order
    of requests and releases, and once everything is released the arena is whole again."""
    from hypothesis import given, settings, strategies as st

    arena = 1 << 20

    @settings(max_examples=60, deadline=None)
    @given(st.lists(st.tuples(st.booleans(), st.integers(1, 200_000), st.integers(0, 1 << 30)), min_size=1, max_size=60))
    def run(ops):
        ctx = cs._C.SymmetricContext(arena_bytes=arena)
        live = []
        for is_alloc, size, pick in ops:
            if is_alloc or not live:
                try:
                    block = ctx.allocate(size)
                except RuntimeError as e:
                    assert "exhausted" in str(e)
                    continue
                off, n = block
                assert off % 256 == 0 and n % 256 == 0 and n >= size and off + n <= arena
                for o, m in live:
                    assert off + n <= o or o + m <= off, (block, (o, m))
                live.append(block)
            else:
                ctx.release(*live.pop(pick % len(live)))
            assert ctx.bytes_in_use() == sum(m for _, m in live)
        for block in live:
            ctx.release(*block)
        assert ctx.bytes_in_use() == 0 and ctx.cached_blocks() == 0
        assert ctx.allocate(arena) == (0, arena)

    run()


@pytest.mark.parametrize("bucket_kb", [1, 64, 1 << 20])
def test_optimizer_overlapped_with_backward_equals_one_step_at_the_end(bucket_kb):
    """With `overlap_optimizer` every bucket of gradients is turned into a parameter update as soon as the backward
    pass has produced it (module::AdamW::step_partial driven by the bucket); the parameters and the optimizer state
    after a few steps are the same as with one whole-model update after the backward pass."""
    from core_scheduler_b200.parallel import GPT2Trainer

    cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=128, padded_vocab_size=128, use_bias=True)
    s = cs.DynamicScheduler(0, device="cpu")
    a = GPT2Trainer(cfg, None, 1, 0, device="cpu", lr=1e-2, bucket_mb=bucket_kb / 1024, scheduler=s, overlap_optimizer=True)
    b = GPT2Trainer(cfg, None, 1, 0, device="cpu", lr=1e-2, scheduler=s, overlap_optimizer=False)
    assert a.bucket is not None and b.bucket is None
    g = torch.Generator().manual_seed(5)
    losses = []
    for _ in range(3):
        ids = torch.randint(0, 128, (2, 33), generator=g)
        x, y = T(ids[:, :-1].contiguous()), T(ids[:, 1:].contiguous())
        la, lb = a.step(x, y), b.step(x, y)
        losses.append((cs.to_torch(s, la).item(), cs.to_torch(s, lb).item()))
    s.synchronize()
    assert all(abs(p - q) < 1e-6 for p, q in losses), losses
    pa_, pb_ = a.model.named_parameters(), b.model.named_parameters()
    for k in pa_:
        assert torch.equal(pa_[k].raw(), pb_[k].raw()), k
    sa, sb = a.optimizer.named_state_tensors(), b.optimizer.named_state_tensors()
    for k in sa:
        assert torch.equal(sa[k].raw(), sb[k].raw()), k
    assert a.optimizer.step_count() == b.optimizer.step_count() == 3
    assert a.bucket.launches() >= 3
